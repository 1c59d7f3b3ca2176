// Fused per-token activation quantization + ternary contraction for small token
// counts (decode).  HBM-bound: the packed weights are streamed once with 128-bit
// loads, expanded in registers and contracted on the int8 tensor path against
// activations quantized into shared memory by the same CTA.
//
// Work decomposition.  A "unit" is 16 weight rows x 512 weights of K (one warp:
// each lane holds 2 x 16 bytes of two rows).  A CTA of 8 warps owns RG row
// tiles (RG in {1,2,4,8}) and splits K over 8/RG warps per tile; partial sums
// meet in a shared-memory int32 tile.  Tokens are processed in groups of
// MT = 8*NT per CTA (grid.y).
//
// Expansion.  In both kernel layouts, (word >> 2p) & 0x03030303 yields four
// weights that are consecutive in K, i.e. the partner of one 32-bit word of int8
// activations.  The activations are scattered into shared memory in the order
// the tensor-core fragments consume them, so the inner loop is layout-agnostic:
// per 16 weights one mask (and, for the single-accumulator variant, one shift)
// and one m16n8k32 u8 x s8 MMA per 8 tokens.  Codes stay unsigned (w + 1); the
// token's sum of activations is subtracted once, in integers, in the epilogue.
// With FOURACC the shift is skipped: the four bit positions accumulate into four
// accumulators scaled by 1, 4, 16, 64 and are combined exactly at the end.
#include "wf_common.cuh"

namespace wf {

constexpr int DEC_THREADS = 256;
constexpr int TOK_STRIDE = 576;  // bytes of shared memory per (k-block, token): 512 + 64 skew (conflict-free 128-bit reads)

struct DecodeParams {
    const void* x;
    int64_t ldx;
    const float* x_scale;  // WF_I8 input only (nullable)
    const uint8_t* codes;
    const float* w_scale;
    float w_scale_host;
    const void* bias;
    int bias_dtype;
    void* y;
    int y_dtype;
    int64_t ldy;
    int32_t* acc_out;
    int M, N, K;
    int KB;   // number of 512-wide k-blocks (K rounded up)
    int RG;   // row tiles per CTA
    int MTA;  // token rows allocated in shared memory per k-block
    int layout;
    float eps;
};

__device__ __forceinline__ void mma_u8s8(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                         uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+r"(d[0]), "+r"(d[1]), "+r"(d[2]), "+r"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint4 ldg_stream(const uint8_t* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
}

// Byte offset, inside the 512-byte region of one (k-block, token), of the 32-bit activation word
// that pairs with (h, t, i, p): half h of the 128-byte weight row segment, lane quarter t, word i of
// the lane's 16 bytes, bit position p.
__device__ __forceinline__ int act_slot(int h, int t, int i, int p) { return (((h * 4 + p) * 4 + t) * 4 + i) * 4; }

// Where the activation word holding k..k+3 (k % 4 == 0, k local to a 512 block) lives.
__device__ __forceinline__ int act_slot_of_k(int layout, int kl) {
    if (layout == WF_LAYOUT_WF16) {
        int aw = kl >> 2;  // 0..127 = 64h + 16t + 4i + p
        return act_slot(aw >> 6, (aw >> 4) & 3, (aw >> 2) & 3, aw & 3);
    }
    // I2_S: block of 128 weights = 32 bytes; byte j holds k = j, j+32, j+64, j+96 at bit positions 3,2,1,0
    int blk = kl >> 7, r = kl & 127, grp = r >> 5, j = r & 31;
    int byte = blk * 32 + j;  // 0..127 within the row segment of this k-block; j % 4 == 0 here
    return act_slot(byte >> 6, (byte >> 4) & 3, (byte >> 2) & 3, 3 - grp);
}

// ---- the quantization prologue: x -> int8 in fragment order, per-token multiplier and sum ----
template <int XDT>
__device__ __forceinline__ void quantize_tokens(const DecodeParams& p, int m0, int m_valid, uint8_t* s_act, float* s_inv,
                                                int* s_rowsum, unsigned* s_maxbits) {
    const int tid = threadIdx.x;
    const int Kp = p.KB * 512;
    // threads per token: all 256 for one token down to one warp per token for 8 or more
    int tpt = DEC_THREADS;
    while (tpt > 32 && DEC_THREADS / tpt < m_valid) tpt >>= 1;
    const int par = DEC_THREADS / tpt;  // tokens handled concurrently
    const int sub = tid / tpt, lane_in = tid % tpt;

    if constexpr (XDT == WF_I8) {
        // already int8: copy into fragment order, sum rows
        for (int tb = 0; tb < m_valid; tb += par) {
            int tok = tb + sub;
            int sum = 0;
            if (tok < m_valid) {
                const int8_t* row = static_cast<const int8_t*>(p.x) + static_cast<int64_t>(m0 + tok) * p.ldx;
                for (int k = lane_in * 16; k < Kp; k += tpt * 16) {
                    uint4 v = make_uint4(0, 0, 0, 0);
                    if (k < p.K) v = __ldg(reinterpret_cast<const uint4*>(row + k));
                    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        sum += __dp4a(static_cast<int>(w[j]), 0x01010101, 0);
                        int kb = (k + 4 * j) >> 9, kl = (k + 4 * j) & 511;
                        *reinterpret_cast<uint32_t*>(s_act + (kb * p.MTA + tok) * TOK_STRIDE + act_slot_of_k(p.layout, kl)) = w[j];
                    }
                }
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
            if (tok < m_valid && (tid & 31) == 0) atomicAdd(&s_rowsum[tok], sum);
        }
        if (tid < m_valid) s_inv[tid] = p.x_scale ? __frcp_rn(p.x_scale[m0 + tid]) : 1.0f;
        return;
    } else {
        // pass 1: absmax per token
        for (int tb = 0; tb < m_valid; tb += par) {
            int tok = tb + sub;
            float mx = 0.f;
            if (tok < m_valid) {
                for (int k = lane_in * 8; k < p.K; k += tpt * 8) {
                    float f[8];
                    load8<XDT>(p.x, static_cast<int64_t>(m0 + tok) * p.ldx + k, f);
#pragma unroll
                    for (int i = 0; i < 8; ++i) mx = fmaxf(mx, fabsf(f[i]));
                }
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
            if (tok < m_valid && (tid & 31) == 0) atomicMax(&s_maxbits[tok], __float_as_uint(mx));
        }
        __syncthreads();
        // pass 2: quantize, scatter, sum
        for (int tb = 0; tb < m_valid; tb += par) {
            int tok = tb + sub;
            int sum = 0;
            if (tok < m_valid) {
                const float s = act_scale_from_absmax<XDT>(__uint_as_float(s_maxbits[tok]), p.eps);
                if (lane_in == 0) s_inv[tok] = __fdiv_rn(1.0f, s);
                for (int k = lane_in * 8; k < Kp; k += tpt * 8) {
                    uint32_t w0 = 0, w1 = 0;
                    if (k < p.K) {
                        float f[8];
                        load8<XDT>(p.x, static_cast<int64_t>(m0 + tok) * p.ldx + k, f);
#pragma unroll
                        for (int i = 0; i < 4; ++i) {
                            int a = quantize_one<XDT>(f[i], s), b = quantize_one<XDT>(f[4 + i], s);
                            sum += a + b;
                            w0 |= static_cast<uint32_t>(a & 0xff) << (8 * i);
                            w1 |= static_cast<uint32_t>(b & 0xff) << (8 * i);
                        }
                    }
                    int kb = k >> 9, kl = k & 511;
                    uint8_t* base = s_act + (kb * p.MTA + tok) * TOK_STRIDE;
                    *reinterpret_cast<uint32_t*>(base + act_slot_of_k(p.layout, kl)) = w0;
                    *reinterpret_cast<uint32_t*>(base + act_slot_of_k(p.layout, kl + 4)) = w1;
                }
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
            if (tok < m_valid && (tid & 31) == 0) atomicAdd(&s_rowsum[tok], sum);
        }
    }
}

struct UnitRegs {
    uint4 r0[2], r1[2];  // [h]: 16 bytes of row g and of row g+8
};

__device__ __forceinline__ void load_unit(const DecodeParams& p, int kb, int row0, int row1, int t, UnitRegs& u) {
    const int64_t rb = p.K >> 2;  // bytes per packed row
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        int64_t off = static_cast<int64_t>(kb) * 128 + h * 64 + t * 16;
        bool kin = off < rb;
        u.r0[h] = (kin && row0 < p.N) ? ldg_stream(p.codes + row0 * rb + off) : make_uint4(0, 0, 0, 0);
        u.r1[h] = (kin && row1 < p.N) ? ldg_stream(p.codes + row1 * rb + off) : make_uint4(0, 0, 0, 0);
    }
}

template <int NT, bool FOURACC>
__device__ __forceinline__ void compute_unit(const UnitRegs& u, const uint8_t* s_act_kb, int MTA, int m_valid, int g, int t,
                                             int (&acc)[NT][FOURACC ? 4 : 1][4]) {
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        const uint32_t wa[4] = {u.r0[h].x, u.r0[h].y, u.r0[h].z, u.r0[h].w};
        const uint32_t wb[4] = {u.r1[h].x, u.r1[h].y, u.r1[h].z, u.r1[h].w};
#pragma unroll
        for (int pp = 0; pp < 4; ++pp) {
            uint32_t a0[4], a1[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                if constexpr (FOURACC) {
                    a0[i] = wa[i] & (0x03030303u << (2 * pp));
                    a1[i] = wb[i] & (0x03030303u << (2 * pp));
                } else {
                    a0[i] = (wa[i] >> (2 * pp)) & 0x03030303u;
                    a1[i] = (wb[i] >> (2 * pp)) & 0x03030303u;
                }
            }
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) {
                const int tok = nt * 8 + g;
                uint4 bw = make_uint4(0, 0, 0, 0);
                if (tok < m_valid)
                    bw = *reinterpret_cast<const uint4*>(s_act_kb + tok * TOK_STRIDE + ((h * 4 + pp) * 4 + t) * 16);
                mma_u8s8(acc[nt][FOURACC ? pp : 0], a0[0], a1[0], a0[1], a1[1], bw.x, bw.y);
                mma_u8s8(acc[nt][FOURACC ? pp : 0], a0[2], a1[2], a0[3], a1[3], bw.z, bw.w);
            }
        }
    }
}

template <int XDT, int NT, bool FOURACC>
__global__ void __launch_bounds__(DEC_THREADS) decode_kernel(const DecodeParams p) {
    extern __shared__ __align__(16) uint8_t smem[];
    constexpr int MT = NT * 8;
    // shared memory: [MT] multipliers, [MT] row sums, [MT] absmax bits, [RG][16][MT] partial sums, activations
    float* s_inv = reinterpret_cast<float*>(smem);
    int* s_rowsum = reinterpret_cast<int*>(smem + MT * 4);
    unsigned* s_maxbits = reinterpret_cast<unsigned*>(smem + MT * 8);
    int* s_red = reinterpret_cast<int*>(smem + MT * 12);
    uint8_t* s_act = smem + MT * 12 + p.RG * 16 * MT * 4;

    // let the next kernel of the stream start its own weight streaming as early as possible
    asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory");

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
    const int rt_local = warp % p.RG, ks = warp / p.RG, KS = 8 / p.RG;
    const int rt = blockIdx.x * p.RG + rt_local;
    const int row0 = rt * 16 + g, row1 = row0 + 8;
    const int m0 = blockIdx.y * MT;
    const int m_valid = min(MT, p.M - m0);

    // weights do not depend on the previous kernel: issue the first unit's loads now
    UnitRegs cur, nxt;
    int kb = ks;
    if (kb < p.KB) load_unit(p, kb, row0, row1, t, cur);

    for (int i = tid; i < MT; i += DEC_THREADS) {
        s_rowsum[i] = 0;
        s_maxbits[i] = 0;
        s_inv[i] = 0.f;
    }
    for (int i = tid; i < p.RG * 16 * MT; i += DEC_THREADS) s_red[i] = 0;
    __syncthreads();

    // x may be produced by the previous kernel of the stream
    asm volatile("griddepcontrol.wait;\n" ::: "memory");
    quantize_tokens<XDT>(p, m0, m_valid, s_act, s_inv, s_rowsum, s_maxbits);
    __syncthreads();

    int acc[NT][FOURACC ? 4 : 1][4];
#pragma unroll
    for (int a = 0; a < NT; ++a)
#pragma unroll
        for (int b = 0; b < (FOURACC ? 4 : 1); ++b)
#pragma unroll
            for (int c = 0; c < 4; ++c) acc[a][b][c] = 0;

#pragma unroll 1
    for (; kb < p.KB; kb += KS) {
        const int kn = kb + KS;
        if (kn < p.KB) load_unit(p, kn, row0, row1, t, nxt);
        compute_unit<NT, FOURACC>(cur, s_act + kb * p.MTA * TOK_STRIDE, p.MTA, m_valid, g, t, acc);
        if (kn < p.KB) cur = nxt;
    }

    // fold the partial sums of the K-splits: lane holds rows g, g+8 x tokens 2t, 2t+1 of every token tile
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
        int v[4];
#pragma unroll
        for (int c = 0; c < 4; ++c) {
            if constexpr (FOURACC)
                v[c] = acc[nt][0][c] + (acc[nt][1][c] >> 2) + (acc[nt][2][c] >> 4) + (acc[nt][3][c] >> 6);
            else
                v[c] = acc[nt][0][c];
        }
        int* base = s_red + rt_local * 16 * MT;
        const int tk = nt * 8 + 2 * t;
        if (KS == 1) {
            base[g * MT + tk] = v[0];
            base[g * MT + tk + 1] = v[1];
            base[(g + 8) * MT + tk] = v[2];
            base[(g + 8) * MT + tk + 1] = v[3];
        } else {
            atomicAdd(&base[g * MT + tk], v[0]);
            atomicAdd(&base[g * MT + tk + 1], v[1]);
            atomicAdd(&base[(g + 8) * MT + tk], v[2]);
            atomicAdd(&base[(g + 8) * MT + tk + 1], v[3]);
        }
    }
    __syncthreads();

    // epilogue: integer correction, fp32 rescale in the stated order, bias, store
    const float s_w = p.w_scale ? __ldg(p.w_scale) : p.w_scale_host;
    const int rows_cta = p.RG * 16;
    for (int idx = tid; idx < rows_cta * m_valid; idx += DEC_THREADS) {
        const int tok = idx / rows_cta, r = idx % rows_cta;
        const int n = blockIdx.x * rows_cta + r;
        if (n >= p.N) continue;
        const int a = s_red[(r >> 4) * 16 * MT + (r & 15) * MT + tok] - s_rowsum[tok];
        float v = rescale(a, s_inv[tok], s_w);
        if (p.bias) v = __fadd_rn(v, load1_rt(p.bias, p.bias_dtype, n));
        const int64_t m = m0 + tok;
        store1_rt(p.y, p.y_dtype, m * p.ldy + n, v);
        if (p.acc_out) p.acc_out[m * p.N + n] = a;
    }
}

template <int XDT, int NT, bool FOURACC>
static int launch_decode(const DecodeParams& p, size_t smem, dim3 grid, unsigned flags, cudaStream_t st) {
    auto kern = decode_kernel<XDT, NT, FOURACC>;
    static thread_local size_t configured = 0;  // per instantiation
    if (smem > 48 * 1024 && smem > configured) {
        WF_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
        configured = smem;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = dim3(DEC_THREADS);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    if (flags & WF_FLAG_PDL) {
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
    }
    WF_CUDA(cudaLaunchKernelEx(&cfg, kern, p));
    return WF_OK;
}

template <int XDT>
static int dispatch_nt(const DecodeParams& p, int NT, size_t smem, dim3 grid, unsigned flags, cudaStream_t st) {
    switch (NT) {
        case 1: return launch_decode<XDT, 1, true>(p, smem, grid, flags, st);
        case 2: return launch_decode<XDT, 2, true>(p, smem, grid, flags, st);
        case 4: return launch_decode<XDT, 4, false>(p, smem, grid, flags, st);
        default: return launch_decode<XDT, 8, false>(p, smem, grid, flags, st);
    }
}

constexpr size_t DEC_SMEM_BUDGET = 200 * 1024;

static size_t decode_smem(int NT, int RG, int KB, int MTA) {
    const int MT = NT * 8;
    return static_cast<size_t>(MT) * 12 + static_cast<size_t>(RG) * 16 * MT * 4 + static_cast<size_t>(KB) * MTA * TOK_STRIDE;
}

}  // namespace wf

using namespace wf;

// Shared argument validation of the two contraction entry points.
int wf_check_linear_args(const char* who, const void* x, int x_dtype, int64_t ldx, const float* x_scale, const uint8_t* codes,
                         int layout, const void* bias, int bias_dtype, void* y, int y_dtype, int64_t ldy, int64_t M, int64_t N,
                         int64_t K) {
    WF_REQUIRE(x && codes && y, "%s: null pointer", who);
    WF_REQUIRE(M > 0 && N > 0 && K > 0, "%s: empty problem (M=%lld N=%lld K=%lld)", who, (long long)M, (long long)N, (long long)K);
    WF_REQUIRE(M < (1 << 24) && N < (1 << 27) && K <= (1 << 16), "%s: dimension too large", who);
    WF_REQUIRE(layout == WF_LAYOUT_WF16 || layout == WF_LAYOUT_I2S, "%s: weights must be in WF16 or I2S layout", who);
    if (layout == WF_LAYOUT_WF16)
        WF_REQUIRE(K % 64 == 0, "%s: K must be a multiple of 64 (K=%lld)", who, (long long)K);
    else
        WF_REQUIRE(K % 128 == 0, "%s: the I2_S layout needs K %% 128 == 0 (K=%lld)", who, (long long)K);
    WF_REQUIRE(x_dtype == WF_I8 || is_float_dtype(x_dtype), "%s: unsupported x dtype %d", who, x_dtype);
    WF_REQUIRE(x_dtype == WF_I8 || x_scale == nullptr, "%s: x_scale is only meaningful with int8 input", who);
    WF_REQUIRE(is_float_dtype(y_dtype), "%s: unsupported y dtype %d", who, y_dtype);
    WF_REQUIRE(!bias || is_float_dtype(bias_dtype), "%s: unsupported bias dtype %d", who, bias_dtype);
    WF_REQUIRE(ldx >= K && ldy >= N, "%s: row strides must cover the rows", who);
    WF_REQUIRE(reinterpret_cast<uintptr_t>(x) % 16 == 0 && (ldx * dtype_size(x_dtype)) % 16 == 0,
               "%s: rows of x must be 16-byte aligned", who);
    WF_REQUIRE(reinterpret_cast<uintptr_t>(codes) % 16 == 0, "%s: codes must be 16-byte aligned", who);
    return WF_OK;
}

extern "C" int wf_bitlinear_decode(const void* x, int x_dtype, int64_t ldx, const float* x_scale, const uint8_t* codes,
                                   int layout, const float* w_scale, float w_scale_host, const void* bias, int bias_dtype,
                                   void* y, int y_dtype, int64_t ldy, int32_t* acc_out, int64_t M, int64_t N, int64_t K,
                                   float eps, unsigned flags, void* stream) {
    if (int rc = wf_check_linear_args("wf_bitlinear_decode", x, x_dtype, ldx, x_scale, codes, layout, bias, bias_dtype, y,
                                      y_dtype, ldy, M, N, K))
        return rc;
    if (int rc = require_device()) return rc;

    DecodeParams p;
    p.x = x; p.ldx = ldx; p.x_scale = x_scale; p.codes = codes; p.w_scale = w_scale; p.w_scale_host = w_scale_host;
    p.bias = bias; p.bias_dtype = bias_dtype; p.y = y; p.y_dtype = y_dtype; p.ldy = ldy; p.acc_out = acc_out;
    p.M = static_cast<int>(M); p.N = static_cast<int>(N); p.K = static_cast<int>(K);
    p.KB = static_cast<int>((K + 511) / 512);
    p.layout = layout; p.eps = eps;

    const int row_tiles = static_cast<int>((N + 15) / 16);
    int RG = row_tiles <= 320 ? 1 : (row_tiles <= 640 ? 2 : (row_tiles <= 1280 ? 4 : 8));
    while (RG < 8 && 8 / RG > p.KB && row_tiles >= 2 * RG) RG <<= 1;  // few k-blocks: give idle warps more rows
    p.RG = RG;

    // tokens per CTA: as many as fit in shared memory, in multiples of 8 up to 64
    int NT = M <= 8 ? 1 : (M <= 16 ? 2 : (M <= 32 ? 4 : 8));
    while (NT > 1 && decode_smem(NT, RG, p.KB, static_cast<int>(M < NT * 8 ? M : NT * 8)) > DEC_SMEM_BUDGET) NT >>= 1;
    const int MT = NT * 8;
    p.MTA = static_cast<int>(M < MT ? M : MT);
    const size_t smem = decode_smem(NT, RG, p.KB, p.MTA);
    if (smem > 227 * 1024) return fail(WF_E_LIMIT, "wf_bitlinear_decode: K=%lld needs %zu bytes of shared memory", (long long)K, smem);

    dim3 grid((row_tiles + RG - 1) / RG, static_cast<unsigned>((M + MT - 1) / MT));
    if (grid.y > 65535) return fail(WF_E_LIMIT, "wf_bitlinear_decode: too many token groups (%u); use wf_bitlinear_prefill", grid.y);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    switch (x_dtype) {
        case WF_F32: return dispatch_nt<WF_F32>(p, NT, smem, grid, flags, st);
        case WF_BF16: return dispatch_nt<WF_BF16>(p, NT, smem, grid, flags, st);
        case WF_F16: return dispatch_nt<WF_F16>(p, NT, smem, grid, flags, st);
        default: return dispatch_nt<WF_I8>(p, NT, smem, grid, flags, st);
    }
}
