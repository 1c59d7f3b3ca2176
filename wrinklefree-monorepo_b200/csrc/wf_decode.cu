// Fused per-token activation quantization + ternary contraction for small token
// counts (decode).  HBM-bound: a persistent kernel streams the packed weights
// once through a ring of shared-memory stages filled by tiled TMA copies (one
// elected producer thread, mbarrier completion; one request brings the
// [k-blocks][16 rows][128 bytes] box of a whole row tile), expands them in registers
// and contracts them on the int8 tensor path against activations that the same
// CTA quantized into shared memory.
//
// Work list.  Every problem (one linear layer applied to M tokens) is cut into
// items of 16*RI weight rows over the whole of K; tokens beyond MT = 8*NT per
// pass form further passes ("chunks") over the same rows.  The items of all
// problems of a launch form one list that is split into contiguous ranges, one
// per CTA, so a CTA quantizes the activations of a problem once and then only
// streams weights.
//
// Inside an item a "unit" is 16 rows x 512 weights of K (a 2 KB tile of the
// stage: 16 rows of 128 bytes), handled by one warp: each lane reads 2 x 16 bytes
// of rows g and g+8.  K is split
// over 16/RI warps per row tile; partial sums meet in a shared-memory int32 tile.
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
//
// Every wait on an mbarrier is bounded: when the bound is hit the CTA records
// WF_E_LIMIT in a device status word, stops waiting anywhere and runs to its end.
#include <cuda.h>
#include <cstddef>

#include "wf_common.cuh"
#include "wf_xchg.cuh"

namespace wf {
__device__ int g_decode_status = 0;
}
#define WF_STATUS_WORD ::wf::g_decode_status
#include "wf_async.cuh"

namespace wf {

constexpr int TILE_BYTES = 2048;  // one unit of packed weights in a stage: 16 rows x 128 bytes
constexpr int DEC_CONSUMERS = 512;               // 16 consumer warps
constexpr int NW = DEC_CONSUMERS / 32;
constexpr int DEC_THREADS = DEC_CONSUMERS + 32;  // + 1 producer warp
constexpr int XCHG_SMEM_OFF = 272;  // shared-memory bytes 272 .. 371: the exchange descriptor of a pushing launch (free in both kernels)
constexpr int TOK_STRIDE = 576;  // bytes of shared memory per (k-block, token): 512 + 64 skew (conflict-free 128-bit reads)
constexpr int MAX_STAGES = 16;

struct DecodeCfg {
    int P;            // problems
    int total_items;
    int RI;           // row tiles (16 rows) per item
    int KBmax;        // k-blocks (512) of the largest K
    int MTA;          // token rows allocated per k-block in shared memory
    int stages;
    int stage_bytes;  // bytes per stage (16*RI rows at the pitch of the largest K)
    int act_off, stage_off;  // byte offsets inside dynamic shared memory
    int nbuf;         // streaming form: activation buffers (2 when they are small, else 1)
    int cpp;          // streaming form: CTAs per problem when ranges are aligned to problems (0: contiguous split)
    int hdr_off;      // two cached descriptor heads
    int wide;         // shared form: every consumer warp takes whole items (all problems read the same x, several items per CTA)
    int items_q, items_r;  // total_items = grid * items_q + items_r
    int uniform_items;     // streaming form: > 0 when all problems have equal M, N, K and layout: items of each
    int x_early;           // ... and problem i reads x at x_base + i * x_stride (bytes), without x_scale
    const void* x_base;
    long long x_stride;
    int x_ready;      // streaming form: x does not depend on the previous kernel; only the stores wait for it
    int ib_off, ib_cap;  // shared-memory copy of the problems' first item indices (searched instead of global memory)
    int decoupled;    // 1: every consumer warp owns whole 16-row items (RI == 1); 0: the 16 warps share each item
    int ss_off;       // per-warp partial sums of squares of the fused RMSNorm input mode: [2][MT][16] floats
    int prefetch;     // some problem names a range to prefetch into L2
    const void* xchg; // the exchange that problems of this launch push their outputs to (wf_problem.xchg), or null
};

template <int NTHREADS = DEC_CONSUMERS>
__device__ __forceinline__ void consumer_sync() {
    asm volatile("bar.sync 1, %0;\n" ::"n"(NTHREADS) : "memory");
}

__device__ __forceinline__ void mma_u8s8(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                         uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+r"(d[0]), "+r"(d[1]), "+r"(d[2]), "+r"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
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


// ---- the quantization stage: x -> int8 in fragment order, per-token multiplier and sum ----
// Executed by the 256 consumer threads together whenever the CTA moves to another (problem, token pass).
// Three phases.  ISSUE starts the reads of x from global memory into registers and returns without using them, so a
// caller can put its first requests for weights behind them (ahead of them, some 100 KB per CTA, the reads of x would
// wait for microseconds).  ABSMAX opens with a barrier (which also publishes a descriptor head that was just copied to
// shared memory) and reduces the absolute maximum per token; int8 input is complete after it.  EMIT opens with a
// barrier, writes the int8 fragments and the sums, and closes with a barrier.
// The first XCache::XC chunks (8 elements each) of a thread's share of the first token group stay in registers from
// ISSUE to EMIT; what lies beyond is read in ABSMAX and again in EMIT.
// `p` supplies the scalar fields (K, ldx, layout, eps); x and x_scale are passed separately.
enum { Q_ISSUE = 0, Q_ABSMAX = 1, Q_EMIT = 2 };
template <int XDT>
struct XCache {
    static constexpr int V = (XDT == WF_F32) ? 2 : 1;   // 16-byte loads per chunk
    static constexpr int XC = (XDT == WF_F32) ? 3 : 6;  // chunks kept
    uint4 r[XC][V];
};
template <int XDT>
__device__ __forceinline__ void load8_raw(const void* base, int64_t elem_off, uint4 (&r)[XCache<XDT>::V]) {
    if constexpr (XDT == WF_F32) {
        const uint4* q = reinterpret_cast<const uint4*>(static_cast<const float*>(base) + elem_off);
        r[0] = __ldg(q);
        r[1] = __ldg(q + 1);
    } else {
        r[0] = __ldg(reinterpret_cast<const uint4*>(static_cast<const uint16_t*>(base) + elem_off));
    }
}
template <int XDT>
__device__ __forceinline__ void decode8(const uint4 (&r)[XCache<XDT>::V], float (&f)[8]) {
    if constexpr (XDT == WF_F32) {
        f[0] = __uint_as_float(r[0].x); f[1] = __uint_as_float(r[0].y); f[2] = __uint_as_float(r[0].z); f[3] = __uint_as_float(r[0].w);
        f[4] = __uint_as_float(r[1].x); f[5] = __uint_as_float(r[1].y); f[6] = __uint_as_float(r[1].z); f[7] = __uint_as_float(r[1].w);
    } else {
        const uint32_t w[4] = {r[0].x, r[0].y, r[0].z, r[0].w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            if constexpr (XDT == WF_BF16) {
                f[2 * i] = __uint_as_float(w[i] << 16);
                f[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
            } else {
                const float2 v = __half22float2(*reinterpret_cast<const __half2*>(&w[i]));
                f[2 * i] = v.x;
                f[2 * i + 1] = v.y;
            }
        }
    }
}

// ---- fused input modes (bf16 only): the activations a projection quantizes are computed on the fly from the
// tensors its unfused predecessor kernel would have read, with that kernel's arithmetic (every intermediate rounded
// to bf16 where the kernel rounds), so the int8 codes equal those of the unfused chain up to the summation order of
// the norm's mean of squares.
//   WF_X_SILU / WF_X_RELU2: x = act(x) * x2            (the gate activation in front of a down projection)
//   WF_X_NORM:              h = x (+ x2);  x = h * rsqrt(mean(h^2) + norm_eps) * norm_w   (residual add + RMSNorm)
__device__ __forceinline__ float rbf(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }
__device__ __forceinline__ float fused_act(float a, int mode) {
    float t;
    if (mode == WF_X_SILU) {
        t = a / (1.0f + __expf(-a));
    } else {
        const float rl = rbf(fmaxf(a, 0.f));
        t = rl * rl;
    }
    return rbf(t);
}
// the residual stream values h = bf16(x + x2) of 8 consecutive k
template <int XDT>
__device__ __forceinline__ void load8_resid(const wf_problem& p, const void* x, int64_t off, float (&f)[8]) {
    load8<XDT>(x, off, f);
    if (p.x2) {
        float d[8];
        load8<XDT>(p.x2, off, d);
#pragma unroll
        for (int i = 0; i < 8; ++i) f[i] = rbf(f[i] + d[i]);
    }
}
// the effective activations of 8 consecutive k of the row that starts at element `base`
template <int XDT>
__device__ __forceinline__ void load8_eff(const wf_problem& p, const void* x, int64_t base, int k, float rnorm, float (&f)[8]) {
    if constexpr (XDT != WF_BF16) {
        load8<XDT>(x, base + k, f);
    } else {
        if (p.x_mode == WF_X_PLAIN) {
            load8<XDT>(x, base + k, f);
        } else if (p.x_mode == WF_X_NORM) {
            load8_resid<XDT>(p, x, base + k, f);
            float w[8];
            load8<XDT>(p.norm_w, k, w);
#pragma unroll
            for (int i = 0; i < 8; ++i) f[i] = rbf(rbf(f[i] * rnorm) * w[i]);
        } else {
            float u[8];
            load8<XDT>(x, base + k, f);
            load8<XDT>(p.x2, base + k, u);
#pragma unroll
            for (int i = 0; i < 8; ++i) f[i] = rbf(fused_act(f[i], p.x_mode) * u[i]);
        }
    }
}

template <int XDT, int NTHREADS, int PHASE>
__device__ __forceinline__ void quantize_phase(const wf_problem& p, const void* x, const float* x_scale, int MTA, int m0, int m_valid,
                                               uint8_t* s_act, float* s_inv, int* s_rowsum, unsigned* s_maxbits, XCache<XDT>& cache,
                                               float* s_ss = nullptr, bool write_h = false) {
    constexpr int XC = XCache<XDT>::XC;
    const int tid = threadIdx.x;
    bool fused = false;  // a fused input mode: the register cache of raw x is not used
    if constexpr (XDT == WF_BF16) fused = p.x_mode != WF_X_PLAIN;
    if constexpr (PHASE == Q_ISSUE) {
        for (int i = tid; i < m_valid; i += NTHREADS) {
            s_rowsum[i] = 0;
            s_maxbits[i] = 0;
        }
    } else {
        consumer_sync<NTHREADS>();
    }
    const int K = p.K, Kp = ((K + 511) >> 9) * 512;
    // threads per token: all of them for one token down to one warp per token for 8 or more
    int tpt = NTHREADS;
    while (tpt > 32 && NTHREADS / tpt < m_valid) tpt >>= 1;
    const int par = NTHREADS / tpt;  // tokens handled concurrently
    const int sub = tid / tpt, lane_in = tid & (tpt - 1);

    if constexpr (XDT == WF_I8) {
        if constexpr (PHASE == Q_ABSMAX) {
            for (int tb = 0; tb < m_valid; tb += par) {
                int tok = tb + sub;
                int sum = 0;
                if (tok < m_valid) {
                    const int8_t* row = static_cast<const int8_t*>(x) + static_cast<int64_t>(m0 + tok) * p.ldx;
                    for (int k = lane_in * 16; k < Kp; k += tpt * 16) {
                        uint4 v = make_uint4(0, 0, 0, 0);
                        if (k < K) v = __ldg(reinterpret_cast<const uint4*>(row + k));
                        const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            sum += __dp4a(static_cast<int>(w[j]), 0x01010101, 0);
                            int kb = (k + 4 * j) >> 9, kl = (k + 4 * j) & 511;
                            *reinterpret_cast<uint32_t*>(s_act + (kb * MTA + tok) * TOK_STRIDE + act_slot_of_k(p.layout, kl)) = w[j];
                        }
                    }
                }
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
                if (tok < m_valid && (tid & 31) == 0) atomicAdd(&s_rowsum[tok], sum);
            }
            if (tid < m_valid) s_inv[tid] = x_scale ? __frcp_rn(x_scale[m0 + tid]) : 1.0f;
        }
    } else {
        if constexpr (PHASE == Q_ISSUE) {
            const int tok = sub;
            if (tok < m_valid && !fused) {
                const int64_t base = static_cast<int64_t>(m0 + tok) * p.ldx;
                int k = lane_in * 8;
#pragma unroll
                for (int c = 0; c < XC; ++c, k += tpt * 8)
                    if (k < K) load8_raw<XDT>(x, base + k, cache.r[c]);
            }
        }
        if constexpr (PHASE == Q_ABSMAX) {
            if constexpr (XDT == WF_BF16) {
                if (p.x_mode == WF_X_NORM) {
                    // mean of squares of the residual stream per token: thread partial over its k in ascending order,
                    // shuffle tree, then the warps' partials are summed in warp order by whoever needs the result
                    for (int tb = 0; tb < m_valid; tb += par) {
                        const int tok = tb + sub;
                        float ss = 0.f;
                        if (tok < m_valid) {
                            const int64_t base = static_cast<int64_t>(m0 + tok) * p.ldx;
                            for (int k = lane_in * 8; k < K; k += tpt * 8) {
                                float f[8];
                                load8_resid<XDT>(p, x, base + k, f);
#pragma unroll
                                for (int i = 0; i < 8; ++i) ss += f[i] * f[i];
                                if (write_h) {  // the updated residual stream, written by one CTA of the launch
                                    uint4 o;
                                    o.x = __bfloat16_as_ushort(__float2bfloat16_rn(f[0])) | (static_cast<uint32_t>(__bfloat16_as_ushort(__float2bfloat16_rn(f[1]))) << 16);
                                    o.y = __bfloat16_as_ushort(__float2bfloat16_rn(f[2])) | (static_cast<uint32_t>(__bfloat16_as_ushort(__float2bfloat16_rn(f[3]))) << 16);
                                    o.z = __bfloat16_as_ushort(__float2bfloat16_rn(f[4])) | (static_cast<uint32_t>(__bfloat16_as_ushort(__float2bfloat16_rn(f[5]))) << 16);
                                    o.w = __bfloat16_as_ushort(__float2bfloat16_rn(f[6])) | (static_cast<uint32_t>(__bfloat16_as_ushort(__float2bfloat16_rn(f[7]))) << 16);
                                    *reinterpret_cast<uint4*>(static_cast<__nv_bfloat16*>(p.h_out) + base + k) = o;
                                }
                            }
                        }
#pragma unroll
                        for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
                        if (tok < m_valid && (tid & 31) == 0) s_ss[tok * 16 + (lane_in >> 5)] = ss;
                    }
                    consumer_sync<NTHREADS>();
                }
            }
            for (int tb = 0; tb < m_valid; tb += par) {
                int tok = tb + sub;
                float mx = 0.f;
                if (tok < m_valid) {
                    const int64_t base = static_cast<int64_t>(m0 + tok) * p.ldx;
                    int k = lane_in * 8;
                    float rnorm = 1.f;
                    if constexpr (XDT == WF_BF16) {
                        if (p.x_mode == WF_X_NORM) {
                            float tot = 0.f;
                            for (int w = 0; w < tpt / 32; ++w) tot += s_ss[tok * 16 + w];
                            rnorm = rsqrtf(tot / static_cast<float>(K) + p.norm_eps);
                        }
                    }
                    if (tb == 0 && !fused) {
#pragma unroll
                        for (int c = 0; c < XC; ++c, k += tpt * 8) {
                            if (k < K) {
                                float f[8];
                                decode8<XDT>(cache.r[c], f);
#pragma unroll
                                for (int i = 0; i < 8; ++i) mx = fmaxf(mx, fabsf(f[i]));
                            }
                        }
                    }
                    // several loads in flight per thread: these are dependent round trips otherwise
#pragma unroll 4
                    for (; k < K; k += tpt * 8) {
                        float f[8];
                        load8_eff<XDT>(p, x, base, k, rnorm, f);
#pragma unroll
                        for (int i = 0; i < 8; ++i) mx = fmaxf(mx, fabsf(f[i]));
                    }
                }
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
                if (tok < m_valid && (tid & 31) == 0) atomicMax(&s_maxbits[tok], __float_as_uint(mx));
            }
        }
        if constexpr (PHASE == Q_EMIT) {
            for (int tb = 0; tb < m_valid; tb += par) {
                int tok = tb + sub;
                int sum = 0;
                if (tok < m_valid) {
                    const float s = act_scale_from_absmax<XDT>(__uint_as_float(s_maxbits[tok]), p.eps);
                    if (lane_in == 0) s_inv[tok] = __fdiv_rn(1.0f, s);
                    const int64_t base = static_cast<int64_t>(m0 + tok) * p.ldx;
                    const int layout = p.layout;
                    auto emit = [&](int k, const float (&f)[8], bool live) {
                        uint32_t w0 = 0, w1 = 0;
                        if (live) {
#pragma unroll
                            for (int i = 0; i < 4; ++i) {
                                int a = quantize_one<XDT>(f[i], s), b = quantize_one<XDT>(f[4 + i], s);
                                sum += a + b;
                                w0 |= static_cast<uint32_t>(a & 0xff) << (8 * i);
                                w1 |= static_cast<uint32_t>(b & 0xff) << (8 * i);
                            }
                        }
                        int kb = k >> 9, kl = k & 511;
                        uint8_t* dst = s_act + (kb * MTA + tok) * TOK_STRIDE;
                        *reinterpret_cast<uint32_t*>(dst + act_slot_of_k(layout, kl)) = w0;
                        *reinterpret_cast<uint32_t*>(dst + act_slot_of_k(layout, kl + 4)) = w1;
                    };
                    int k = lane_in * 8;
                    float rnorm = 1.f;
                    if constexpr (XDT == WF_BF16) {
                        if (p.x_mode == WF_X_NORM) {
                            float tot = 0.f;
                            for (int w = 0; w < tpt / 32; ++w) tot += s_ss[tok * 16 + w];
                            rnorm = rsqrtf(tot / static_cast<float>(K) + p.norm_eps);
                        }
                    }
                    if (tb == 0 && !fused) {
#pragma unroll
                        for (int c = 0; c < XC; ++c, k += tpt * 8) {
                            if (k < Kp) {
                                float f[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
                                if (k < K) decode8<XDT>(cache.r[c], f);
                                emit(k, f, k < K);
                            }
                        }
                    }
#pragma unroll 4
                    for (; k < Kp; k += tpt * 8) {
                        float f[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
                        if (k < K) load8_eff<XDT>(p, x, base, k, rnorm, f);
                        emit(k, f, k < K);
                    }
                }
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
                if (tok < m_valid && (tid & 31) == 0) atomicAdd(&s_rowsum[tok], sum);
            }
        }
    }
    if constexpr (PHASE == Q_EMIT) consumer_sync<NTHREADS>();
}

// All three phases in a row.  The caller has made the fields of `p` visible (a barrier after copying a head).
template <int XDT, int NTHREADS = DEC_CONSUMERS>
__device__ __forceinline__ void quantize_tokens(const wf_problem& p, int MTA, int m0, int m_valid, uint8_t* s_act, float* s_inv,
                                                int* s_rowsum, unsigned* s_maxbits, float* s_ss, bool write_h) {
    XCache<XDT> cache;
    const void* x = p.x;
    const float* xs = p.x_scale;
    quantize_phase<XDT, NTHREADS, Q_ISSUE>(p, x, xs, MTA, m0, m_valid, s_act, s_inv, s_rowsum, s_maxbits, cache, s_ss, write_h);
    quantize_phase<XDT, NTHREADS, Q_ABSMAX>(p, x, xs, MTA, m0, m_valid, s_act, s_inv, s_rowsum, s_maxbits, cache, s_ss, write_h);
    quantize_phase<XDT, NTHREADS, Q_EMIT>(p, x, xs, MTA, m0, m_valid, s_act, s_inv, s_rowsum, s_maxbits, cache, s_ss, write_h);
}

__device__ __forceinline__ uint4 lds128(uint32_t addr) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];\n" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
    return v;
}

// One unit: 16 rows x 512 weights from the stage (rows g and g+8 of the tile, 2 x 16 bytes each per lane)
// against the activations of one k-block.
// Order matters more than count here.  The MMAs of one accumulator are a dependent chain (about 35 cycles each), and
// the shared-memory loads are volatile statements that the compiler keeps where they are written: a load directly in
// front of the MMA that uses it, followed by a second MMA on the same accumulator, serialises a unit into sixteen
// round trips (measured: 717 cycles per unit, 45 per MMA, the warp idle in between).  So every load of a unit is
// issued before its first MMA, and consecutive MMAs go to different accumulators.
template <int NT, bool FOURACC>
__device__ __forceinline__ void compute_unit(uint32_t w_r0, uint32_t w_r1, uint32_t s_act_kb, int m_valid, int g, int t,
                                             int (&acc)[NT][FOURACC ? 4 : 1][4]) {
    auto code = [](uint32_t w, int pp) -> uint32_t {
        if constexpr (FOURACC)
            return w & (0x03030303u << (2 * pp));
        else
            return (w >> (2 * pp)) & 0x03030303u;
    };
    if constexpr (NT == 1) {
        uint4 ra[2], rb[2], bw[2][4];
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            ra[h] = lds128(w_r0 + h * 64 + t * 16);
            rb[h] = lds128(w_r1 + h * 64 + t * 16);
        }
        const bool tok_ok = g < m_valid;
#pragma unroll
        for (int h = 0; h < 2; ++h)
#pragma unroll
            for (int pp = 0; pp < 4; ++pp) {
                bw[h][pp] = make_uint4(0, 0, 0, 0);
                if (tok_ok) bw[h][pp] = lds128(s_act_kb + g * TOK_STRIDE + ((h * 4 + pp) * 4 + t) * 16);
            }
        if constexpr (FOURACC) {
#pragma unroll
            for (int h = 0; h < 2; ++h) {
#pragma unroll
                for (int pp = 0; pp < 4; ++pp)
                    mma_u8s8(acc[0][pp], code(ra[h].x, pp), code(rb[h].x, pp), code(ra[h].y, pp), code(rb[h].y, pp), bw[h][pp].x, bw[h][pp].y);
#pragma unroll
                for (int pp = 0; pp < 4; ++pp)
                    mma_u8s8(acc[0][pp], code(ra[h].z, pp), code(rb[h].z, pp), code(ra[h].w, pp), code(rb[h].w, pp), bw[h][pp].z, bw[h][pp].w);
            }
        } else {  // one accumulator: four partial sums of the unit keep the chains apart
            int part[4][4] = {};
#pragma unroll
            for (int h = 0; h < 2; ++h) {
#pragma unroll
                for (int pp = 0; pp < 4; ++pp)
                    mma_u8s8(part[pp], code(ra[h].x, pp), code(rb[h].x, pp), code(ra[h].y, pp), code(rb[h].y, pp), bw[h][pp].x, bw[h][pp].y);
#pragma unroll
                for (int pp = 0; pp < 4; ++pp)
                    mma_u8s8(part[pp], code(ra[h].z, pp), code(rb[h].z, pp), code(ra[h].w, pp), code(rb[h].w, pp), bw[h][pp].z, bw[h][pp].w);
            }
#pragma unroll
            for (int c = 0; c < 4; ++c) acc[0][0][c] += (part[0][c] + part[1][c]) + (part[2][c] + part[3][c]);
        }
    } else {
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const uint4 ra = lds128(w_r0 + h * 64 + t * 16);
            const uint4 rb = lds128(w_r1 + h * 64 + t * 16);
#pragma unroll
            for (int pp = 0; pp < 4; ++pp) {
                const uint32_t a0 = code(ra.x, pp), a1 = code(rb.x, pp), a2 = code(ra.y, pp), a3 = code(rb.y, pp);
                const uint32_t c0 = code(ra.z, pp), c1 = code(rb.z, pp), c2 = code(ra.w, pp), c3 = code(rb.w, pp);
                constexpr int NG = NT < 4 ? NT : 4;  // token tiles whose activations are in registers at a time
#pragma unroll
                for (int n0 = 0; n0 < NT; n0 += NG) {
                    uint4 bw[NG];
#pragma unroll
                    for (int nt = 0; nt < NG; ++nt) {
                        const int tok = (n0 + nt) * 8 + g;
                        bw[nt] = make_uint4(0, 0, 0, 0);
                        if (tok < m_valid) bw[nt] = lds128(s_act_kb + tok * TOK_STRIDE + ((h * 4 + pp) * 4 + t) * 16);
                    }
#pragma unroll
                    for (int nt = 0; nt < NG; ++nt) mma_u8s8(acc[n0 + nt][FOURACC ? pp : 0], a0, a1, a2, a3, bw[nt].x, bw[nt].y);
#pragma unroll
                    for (int nt = 0; nt < NG; ++nt) mma_u8s8(acc[n0 + nt][FOURACC ? pp : 0], c0, c1, c2, c3, bw[nt].z, bw[nt].w);
                }
            }
        }
    }
}


// One K segment of one 16-row tile -> `dst` (consecutive 2 KB tiles, one per 512-weight block of the segment).
// Returns the bytes that will arrive.  Segment s covers blocks [s * _kb_seg, min(KB, (s + 1) * _kb_seg)); full
// blocks come through the 3-D view (box of _kb_seg blocks, or the shorter box of the last segment), the partial
// last block of K through its own 2-D view.
__device__ __forceinline__ unsigned segment_bytes(const wf_problem* p, int seg) {
    const int KB = (p->K + 511) >> 9;
    const int lo = seg * p->_kb_seg;
    const int n = min(KB - lo, p->_kb_seg);
    return static_cast<unsigned>(n) * TILE_BYTES;
}
// `h` supplies the scalar fields (it may be a copy of the descriptor's head in shared memory), `gp` the tensor maps,
// which the TMA unit reads from global memory.
__device__ __forceinline__ void issue_segment(const wf_problem* h, const wf_problem* gp, int row, int seg, uint8_t* dst, uint64_t* bar) {
    const int KB = (h->K + 511) >> 9, kbf = h->_kb_full, lo = seg * h->_kb_seg;
    const int n = min(KB - lo, h->_kb_seg);
    if (kbf > 0) {
        const int nfull = max(0, min(kbf - lo, h->_kb_seg));
        if (nfull == h->_kb_seg)
            tma_load_3d(dst, gp->_tmap_main, 0, row, lo, bar);
        else if (nfull > 0)
            tma_load_3d(dst, gp->_tmap_last, 0, row, lo, bar);
        if (nfull < n) tma_load_2d(dst + nfull * TILE_BYTES, gp->_tmap_tail, 0, row, bar);  // the partial block of K
    } else {  // plain 2-D view: one request per 128-byte column block
        for (int i = 0; i < n; ++i) tma_load_2d(dst + i * TILE_BYTES, gp->_tmap_tail, (lo + i) * 128, row, bar);
    }
}
__device__ __forceinline__ void issue_segment(const wf_problem* p, int row, int seg, uint8_t* dst, uint64_t* bar) {
    issue_segment(p, p, row, seg, dst, bar);
}

// ---- the head of a descriptor, cached in shared memory -------------------------------------------------
// Every read of a descriptor field from global memory is a round trip of half a microsecond, and a barrier
// makes the compiler repeat it.  The CTA therefore copies the head (all fields before the tensor maps) of the
// problem it works on into shared memory once, together with the VALUE of the weight scale.
constexpr int HDR_WORDS = 42;    // 168 bytes: up to and including the fused-input fields
constexpr int HDR_STRIDE = 192;  // bytes per cached head; word HDR_WORDS holds the weight scale
static_assert(offsetof(wf_problem, prefetch) == HDR_WORDS * 4 && offsetof(wf_problem, _tmap_main) >= HDR_WORDS * 4, "head of wf_problem");

__device__ __forceinline__ void fill_header(uint8_t* slot, const wf_problem* src, int t) {
    uint32_t* dst = reinterpret_cast<uint32_t*>(slot);
    if (static_cast<unsigned>(t) < static_cast<unsigned>(HDR_WORDS))
        dst[t] = reinterpret_cast<const uint32_t*>(src)[t];
    else if (t == HDR_WORDS)
        dst[HDR_WORDS] = __float_as_uint(src->w_scale ? __ldg(src->w_scale) : src->w_scale_host);
}
__device__ __forceinline__ float header_w_scale(const uint8_t* slot) {
    return __uint_as_float(reinterpret_cast<const uint32_t*>(slot)[HDR_WORDS]);
}

// item index -> (problem, token pass, row item)
// `ib` is the shared-memory table of _item_begin (valid for the first ib_cap problems): a search through global memory
// is a chain of dependent cache misses, several microseconds per call.
// `uni` > 0: every problem of the group has that many items (a stack of equal layers), no table is needed.
__device__ __forceinline__ int first_item(const wf_problem* __restrict__ probs, int pi, const int* ib, int ib_cap, int uni = 0) {
    if (uni > 0) return pi * uni;
    return pi < ib_cap ? ib[pi] : probs[pi]._item_begin;
}
// item index -> problem, and the item's index inside the problem
__device__ __forceinline__ int locate_problem(const wf_problem* __restrict__ probs, int P, int item, const int* ib, int ib_cap, int& local,
                                              int uni = 0) {
    if (uni > 0) {
        const int pi = item / uni;
        local = item - pi * uni;
        return pi;
    }
    int lo = 0, hi = P - 1;
    while (lo < hi) {  // last problem whose first item <= item
        int mid = (lo + hi + 1) >> 1;
        if (first_item(probs, mid, ib, ib_cap) <= item) lo = mid; else hi = mid - 1;
    }
    local = item - first_item(probs, lo, ib, ib_cap);
    return lo;
}
__device__ __forceinline__ void locate_item(const wf_problem* __restrict__ probs, int P, int item, int& pi, int& chunk, int& ritem,
                                            const int* ib, int ib_cap) {
    int local;
    pi = locate_problem(probs, P, item, ib, ib_cap, local);
    const int row_items = probs[pi]._row_items;
    chunk = local / row_items;
    ritem = local % row_items;
}

// Asks L2 for this CTA's share of every problem's prefetch range (see wf_problem.prefetch); thread `tid` of `nthreads`.
__device__ __forceinline__ void issue_l2_prefetch(const wf_problem* __restrict__ probs, int P, int tid, int nthreads) {
    constexpr long long PIECE = 16384;  // bytes per instruction
    for (int i = 0; i < P; ++i) {
        const char* base = static_cast<const char*>(probs[i].prefetch);
        const long long bytes = probs[i].prefetch_bytes;
        if (!base || bytes <= 0) continue;
        const long long per = ((bytes + gridDim.x - 1) / gridDim.x + 15) / 16 * 16;
        const long long lo = per * blockIdx.x, hi = lo + per < bytes ? lo + per : bytes;
        for (long long o = lo + static_cast<long long>(tid) * PIECE; o < hi; o += static_cast<long long>(nthreads) * PIECE) {
            const unsigned n = static_cast<unsigned>(hi - o < PIECE ? hi - o : PIECE);
            asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;\n" ::"l"(base + o), "r"(n) : "memory");
        }
    }
}

// The push side of a fused exchange: copies what this CTA has produced (the items [beg, end) of the work list; rows_item
// rows each) from its local outputs into every rank's exchange buffer and reports the number of elements.  Called by the
// `nthreads` threads that made the stores, after all of them have passed a barrier.  Consecutive items of one (problem,
// token pass) go out as one block of rows.  A CTA without work has nothing to report.
template <int NTHREADS>
__device__ __forceinline__ void xchg_push_items(const DecodeCfg& cfg, const wf_problem* __restrict__ probs, int beg, int end, int rows_item,
                                                const int* s_ib, int uni, int tid, const uint8_t* s_xchg) {
    const wf_xchg* x = reinterpret_cast<const wf_xchg*>(s_xchg);  // fetched into shared memory at the kernel's start
    const unsigned step = *reinterpret_cast<const unsigned*>(s_xchg + 96) + 1;
    unsigned elems = 0;
    for (int it = beg; it < end;) {
        int local;
        const int pi = locate_problem(probs, cfg.P, it, s_ib, cfg.ib_cap, local, uni);
        const wf_problem* q = &probs[pi];
        const int row_items = q->_row_items, chunk = local / row_items, ritem = local % row_items;
        const int run = min(end - it, row_items - ritem);
        const int64_t bytes = static_cast<int64_t>(q->M) * q->N * 2;
        if (q->xchg != nullptr && static_cast<uint64_t>(bytes) <= x->slot_bytes) {
            const int m0 = chunk * cfg.MTA, m1 = min(q->M, m0 + cfg.MTA);
            const int r0 = ritem * rows_item, r1 = min(q->N, (ritem + run) * rows_item);
            xchg_push_block(x, step, static_cast<const uint16_t*>(q->y), q->ldy, q->N, m0, m1, r0, r1, tid, NTHREADS);
            elems += static_cast<unsigned>((m1 - m0) * (r1 - r0));
        }
        it += run;
    }
    if (elems == 0) return;  // uniform over the CTA
    asm volatile("bar.sync 3, %0;\n" ::"n"(NTHREADS) : "memory");  // every thread's peer stores are issued
    if (tid == 0) xchg_report(x, step, elems);
}

template <int XDT, int NT, bool FOURACC>
__global__ void __launch_bounds__(DEC_THREADS, 1)
    decode_kernel(const wf_problem* __restrict__ dev_problems, const __grid_constant__ wf_problem single, const DecodeCfg cfg) {
    extern __shared__ __align__(128) uint8_t smem[];
    constexpr int MT = NT * 8;
    uint64_t* full = reinterpret_cast<uint64_t*>(smem);
    uint64_t* empty = full + MAX_STAGES;
    volatile int* poisoned = reinterpret_cast<volatile int*>(smem + 256);
    float* s_inv = reinterpret_cast<float*>(smem + 384);
    int* s_rowsum = reinterpret_cast<int*>(smem + 384 + MT * 4);
    unsigned* s_maxbits = reinterpret_cast<unsigned*>(smem + 384 + MT * 8);
    int* s_red = reinterpret_cast<int*>(smem + 384 + MT * 12);  // two buffers of RI*16*MT
    uint8_t* s_act = smem + cfg.act_off;
    uint8_t* s_stage = smem + cfg.stage_off;
    const wf_problem* probs = dev_problems ? dev_problems : &single;

    // let the next kernel of the stream start its own weight streaming as early as possible
    asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory");

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int red_size = cfg.RI * 16 * MT;
    if (tid == 0) {
        for (int s = 0; s < cfg.stages; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], cfg.wide ? 1 : NW);
        }
        *poisoned = 0;
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
    for (int i = tid; i < 2 * red_size; i += DEC_THREADS) s_red[i] = 0;
    int* s_ib = reinterpret_cast<int*>(smem + cfg.ib_off);
    for (int i = tid; i < cfg.ib_cap; i += DEC_THREADS) s_ib[i] = probs[i]._item_begin;
    __syncthreads();

    // an even split of the item list: the first items_r CTAs take one item more
    const int bx = blockIdx.x;
    const int beg = bx * cfg.items_q + min(bx, cfg.items_r);
    const int end = beg + cfg.items_q + (bx < cfg.items_r ? 1 : 0);
    const int rows_item = cfg.RI * 16;

    if (warp == DEC_CONSUMERS / 32) {
        // ---------------- producer: weights do not depend on the previous kernel, stream them right away
        // The item list is walked incrementally: one search at the start, then only counters.
        int pi, chunk, ritem;
        locate_item(probs, cfg.P, beg, pi, chunk, ritem, s_ib, cfg.ib_cap);
        // Only one lane streams: a whole 16-row tile over all of K is one TMA request (plus one for a K tail).  The other
        // lanes ask L2 for the ranges the problems name (the next launch's weights), beside the stream.
        if (lane != 0 && cfg.prefetch) issue_l2_prefetch(probs, cfg.P, lane - 1, 31);
        if (lane == 0) {
            const wf_problem* p = &probs[pi];
            int N = p->N, row_items = p->_row_items, chunks = p->_chunks;
            int KB = (p->K + 511) >> 9;
            for (int it = beg, n = 0; it < end; ++it, ++n) {
                const int stage = n % cfg.stages;
                if (n >= cfg.stages) mbar_wait(&empty[stage], ((n / cfg.stages) - 1) & 1, poisoned);
                const int r0 = ritem * rows_item;
                int tiles = (N - r0 + 15) >> 4;
                tiles = tiles < cfg.RI ? tiles : cfg.RI;
                mbar_expect_tx(&full[stage], static_cast<unsigned>(tiles * KB) * TILE_BYTES);
                uint8_t* dst = s_stage + static_cast<size_t>(stage) * cfg.stage_bytes;
                for (int rt = 0; rt < tiles; ++rt, dst += KB * TILE_BYTES)
                    for (int seg = 0; seg < p->_ksegs; ++seg)
                        issue_segment(p, r0 + rt * 16, seg, dst + seg * p->_kb_seg * TILE_BYTES, &full[stage]);
                if (++ritem == row_items) {
                    ritem = 0;
                    if (++chunk == chunks) {
                        chunk = 0;
                        if (++pi < cfg.P) {
                            p = &probs[pi];
                            N = p->N; row_items = p->_row_items; chunks = p->_chunks;
                            KB = (p->K + 511) >> 9;
                        }
                    }
                }
            }
        }
        return;
    }

    // ---------------- consumers
    const int g = lane >> 2, t = lane & 3;
    const int rt_local = warp % cfg.RI, ks = warp / cfg.RI, KS = NW / cfg.RI;
    uint8_t* s_hdr = smem + cfg.hdr_off;
    const wf_problem& p = *reinterpret_cast<const wf_problem*>(s_hdr);  // head of the current problem (no tensor maps)
    int hdr_p = -1, cur_p = -1, cur_chunk = -1, m0 = 0, m_valid = 0;
    if (beg < end) {  // the descriptor does not depend on the previous kernel: fetch its head before waiting
        int local;
        hdr_p = locate_problem(probs, cfg.P, beg, s_ib, cfg.ib_cap, local);
        fill_header(s_hdr, &probs[hdr_p], tid);
    }
    // x may be produced by the previous kernel of the stream
    asm volatile("griddepcontrol.wait;\n" ::: "memory");
    uint8_t* const s_xchg = smem + XCHG_SMEM_OFF;
    if (cfg.xchg) xchg_fetch_async(cfg.xchg, s_xchg, tid);  // used at the end
    consumer_sync();

    if (cfg.wide) {
        // Every problem of the group reads the same tokens and a CTA has several items: x is quantized once, then
        // each warp takes whole items (all of K, epilogue from its own accumulators) and nothing synchronises the CTA
        // any more.  With all 16 warps on one item at a time, the two barriers and the shared-memory reduction per
        // item (about 0.7 us) made a 29 MB gate/up launch compute-latency-bound.
        if (beg >= end) {
            if (cfg.xchg) xchg_fetch_wait(tid);  // no copy is left in flight
            return;
        }
        const int m_all = min(cfg.MTA, p.M);
        {
            int local_first;
            locate_problem(probs, cfg.P, beg, s_ib, cfg.ib_cap, local_first);
            quantize_tokens<XDT>(p, cfg.MTA, 0, m_all, s_act, s_inv, s_rowsum, s_maxbits, reinterpret_cast<float*>(smem + cfg.ss_off),
                                 p.h_out != nullptr && local_first == 0);
        }
        const uint32_t act0 = smem_u32(s_act);
        const int KB = (p.K + 511) >> 9;
        // Warp w owns stage w and takes the items w, w + W, ... (W = stages <= 16 warps): a barrier is then always waited
        // on by the same warp, phase after phase.  (A warp that waits for a later phase of a barrier whose current phase
        // has not completed would pass at once: the parity of the wait only tells two consecutive phases apart.)
        const int W = cfg.stages;
        for (int n = warp; warp < W && n < end - beg; n += W) {
            int local;
            const int pi = locate_problem(probs, cfg.P, beg + n, s_ib, cfg.ib_cap, local);
            const wf_problem* hp = pi == hdr_p ? &p : &probs[pi];
            const int my_row = local * 16;  // one pass of tokens: the item index is the row item
            const int N = hp->N, y_dtype = hp->y_dtype, bias_dtype = hp->bias_dtype;
            const float s_w = hp->w_scale ? __ldg(hp->w_scale) : hp->w_scale_host;
            void* const y = hp->y;
            const void* const bias = hp->bias;
            int32_t* const acc_out = hp->acc_out;
            const int64_t ldy = hp->ldy;
            const int stage = warp;
            mbar_wait(&full[stage], (n / W) & 1, poisoned);
            int acc[NT][FOURACC ? 4 : 1][4];
#pragma unroll
            for (int a = 0; a < NT; ++a)
#pragma unroll
                for (int b = 0; b < (FOURACC ? 4 : 1); ++b)
#pragma unroll
                    for (int c = 0; c < 4; ++c) acc[a][b][c] = 0;
            const uint32_t w_r0 = smem_u32(s_stage) + stage * cfg.stage_bytes + g * 128;
#pragma unroll 1
            for (int kb = 0; kb < KB; ++kb)
                compute_unit<NT, FOURACC>(w_r0 + kb * TILE_BYTES, w_r0 + kb * TILE_BYTES + 1024, act0 + kb * cfg.MTA * TOK_STRIDE, m_all, g, t,
                                          acc);
            __syncwarp();
            if (lane == 0) mbar_arrive(&empty[stage]);  // the stage has been read
            const int row_a = my_row + g, row_b = row_a + 8;
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) {
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    int v;
                    if constexpr (FOURACC)
                        v = acc[nt][0][c] + (acc[nt][1][c] >> 2) + (acc[nt][2][c] >> 4) + (acc[nt][3][c] >> 6);
                    else
                        v = acc[nt][0][c];
                    const int tok = nt * 8 + 2 * t + (c & 1);
                    const int nrow = (c & 2) ? row_b : row_a;
                    if (tok < m_all && nrow < N) {
                        const int a = v - s_rowsum[tok];
                        float out = rescale(a, s_inv[tok], s_w);
                        if (bias) out = __fadd_rn(out, load1_rt(bias, bias_dtype, nrow));
                        store1_rt(y, y_dtype, static_cast<int64_t>(tok) * ldy + nrow, out);
                        if (acc_out) acc_out[static_cast<int64_t>(tok) * N + nrow] = a;
                    }
                }
            }
        }
        if (cfg.xchg) {
            xchg_fetch_wait(tid);
            consumer_sync();  // every warp's outputs are written
            xchg_push_items<DEC_CONSUMERS>(cfg, probs, beg, end, rows_item, s_ib, 0, tid, s_xchg);
        }
        return;
    }

    for (int it = beg, n = 0; it < end; ++it, ++n) {
        int local;
        const int pi = locate_problem(probs, cfg.P, it, s_ib, cfg.ib_cap, local);
        if (pi != hdr_p) {
            consumer_sync();  // nobody still reads the previous head
            fill_header(s_hdr, &probs[pi], tid);
            hdr_p = pi;
            consumer_sync();
        }
        const int chunk = local / p._row_items, ritem = local % p._row_items;
        if (pi != cur_p || chunk != cur_chunk) {
            consumer_sync();  // nobody still reads the multipliers / sums of the previous pass
            cur_p = pi;
            cur_chunk = chunk;
            m0 = chunk * cfg.MTA;
            m_valid = min(cfg.MTA, p.M - m0);
            quantize_tokens<XDT>(p, cfg.MTA, m0, m_valid, s_act, s_inv, s_rowsum, s_maxbits, reinterpret_cast<float*>(smem + cfg.ss_off),
                                 p.h_out != nullptr && ritem == 0);
        }
        const int stage = n % cfg.stages;
        mbar_wait(&full[stage], (n / cfg.stages) & 1, poisoned);

        int acc[NT][FOURACC ? 4 : 1][4];
#pragma unroll
        for (int a = 0; a < NT; ++a)
#pragma unroll
            for (int b = 0; b < (FOURACC ? 4 : 1); ++b)
#pragma unroll
                for (int c = 0; c < 4; ++c) acc[a][b][c] = 0;

        const int KB = (p.K + 511) >> 9;
        const uint32_t w_r0 = smem_u32(s_stage) + stage * cfg.stage_bytes + rt_local * KB * TILE_BYTES + g * 128;
        const uint32_t act0 = smem_u32(s_act);
#pragma unroll 1
        for (int kb = ks; kb < KB; kb += KS)
            compute_unit<NT, FOURACC>(w_r0 + kb * TILE_BYTES, w_r0 + kb * TILE_BYTES + 1024, act0 + kb * cfg.MTA * TOK_STRIDE,
                                      m_valid, g, t, acc);
        __syncwarp();
        if (lane == 0) mbar_arrive(&empty[stage]);  // this warp no longer reads the stage

        // fold the partial sums of the K-splits: lane holds rows g, g+8 x tokens 2t, 2t+1 of every token tile
        int* red = s_red + (n & 1) * red_size + rt_local * 16 * MT;
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
            const int tk = nt * 8 + 2 * t;
            atomicAdd(&red[g * MT + tk], v[0]);
            atomicAdd(&red[g * MT + tk + 1], v[1]);
            atomicAdd(&red[(g + 8) * MT + tk], v[2]);
            atomicAdd(&red[(g + 8) * MT + tk + 1], v[3]);
        }
        consumer_sync();

        // epilogue: integer correction, fp32 rescale in the stated order, bias, store; clears the tile
        const float s_w = header_w_scale(s_hdr);
        int* redb = s_red + (n & 1) * red_size;
        const int r0 = ritem * rows_item;
        for (int idx = tid; idx < rows_item * m_valid; idx += DEC_CONSUMERS) {
            const int tok = idx / rows_item, r = idx % rows_item;
            const int cell = (r >> 4) * 16 * MT + (r & 15) * MT + tok;
            const int raw = redb[cell];
            redb[cell] = 0;
            const int nrow = r0 + r;
            if (nrow >= p.N) continue;
            const int a = raw - s_rowsum[tok];
            float v = rescale(a, s_inv[tok], s_w);
            if (p.bias) v = __fadd_rn(v, load1_rt(p.bias, p.bias_dtype, nrow));
            const int64_t m = m0 + tok;
            store1_rt(p.y, p.y_dtype, m * p.ldy + nrow, v);
            if (p.acc_out) p.acc_out[m * p.N + nrow] = a;
        }
    }
    if (cfg.xchg) {
        xchg_fetch_wait(tid);
        consumer_sync();  // every thread's outputs are written
        xchg_push_items<DEC_CONSUMERS>(cfg, probs, beg, end, rows_item, s_ib, 0, tid, s_xchg);
    }
}

// ---- streaming form: every warp owns one stage and is its own producer ------------------------------
// Used when a launch has thousands of 16-row items.  CTAs are half-size (8 warps, at most half of an SM's
// shared memory) so that two are resident per SM: the prologue and the tail of one overlap the streaming of
// the other, also across launches chained with programmatic dependent launch.  Warp w consumes the items
// w, w + S, w + 2S, ... of the CTA's range (S = stages <= 8 warps); as soon as its MMA loop has read the stage it issues the TMA
// request of its next item itself, so no thread serialises the requests of the CTA and no "empty"
// barrier exists.  The CTA only synchronises where it moves to another (problem, token pass).
struct ItemCursor {  // walks the item list in strides
    int pi, chunk, ritem, row_items, chunks;
};

constexpr int STREAM_THREADS = 256;  // 8 warps; two such CTAs share an SM
constexpr int SW = STREAM_THREADS / 32;

template <int XDT, int NT, bool FOURACC>
__global__ void __launch_bounds__(STREAM_THREADS, 2)
    decode_stream_kernel(const wf_problem* __restrict__ dev_problems, const __grid_constant__ wf_problem single, const DecodeCfg cfg) {
    extern __shared__ __align__(128) uint8_t smem[];
    constexpr int MT = NT * 8;
    uint64_t* full = reinterpret_cast<uint64_t*>(smem);
    volatile int* poisoned = reinterpret_cast<volatile int*>(smem + 256);
    float* s_inv = reinterpret_cast<float*>(smem + 384);                    // [2][MT]
    int* s_rowsum = reinterpret_cast<int*>(smem + 384 + MT * 8);            // [2][MT]
    unsigned* s_maxbits = reinterpret_cast<unsigned*>(smem + 384 + MT * 16);  // [2][MT]
    uint8_t* s_act = smem + cfg.act_off;                                    // [2][KBmax * MTA * TOK_STRIDE]
    uint8_t* s_stage = smem + cfg.stage_off;
    uint8_t* s_hdr = smem + cfg.hdr_off;                                    // [2][HDR_STRIDE], one per activation buffer
    float* const s_ss = reinterpret_cast<float*>(smem + cfg.ss_off);                        // [2][MT * 16]
    int* s_ib = reinterpret_cast<int*>(smem + cfg.ib_off);
    const wf_problem* probs = dev_problems ? dev_problems : &single;

    asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory");
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
    const int S = cfg.stages;

    if (tid == 0) {
        for (int s = 0; s < S; ++s) mbar_init(&full[s], 1);
        *poisoned = 0;
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
    // A stack of equal problems needs no table of first items, and the scalar fields of every descriptor equal those
    // of the copy that travels as a kernel parameter: the first requests for weights go out without any read of
    // global memory before them.
    const int uni = cfg.uniform_items;
    if (uni == 0)
        for (int i = tid; i < cfg.ib_cap; i += STREAM_THREADS) s_ib[i] = probs[i]._item_begin;
    __syncthreads();

    // The CTA's range of items: an even share of one problem when the grid divides well over the problems
    // (one quantization per CTA, no pass boundary inside a range), else an even share of the whole list.
    int beg, end;
    if (cfg.cpp > 0) {
        const int pi = blockIdx.x / cfg.cpp, sub = blockIdx.x % cfg.cpp;
        if (pi >= cfg.P) return;
        const int ib = first_item(probs, pi, s_ib, cfg.ib_cap, uni);
        const int cnt = (pi + 1 < cfg.P ? first_item(probs, pi + 1, s_ib, cfg.ib_cap, uni) : cfg.total_items) - ib;
        const int q = cnt / cfg.cpp, r = cnt - q * cfg.cpp;  // the first r CTAs of the problem take one item more
        beg = ib + sub * q + min(sub, r);
        end = beg + q + (sub < r ? 1 : 0);
    } else {
        const int bx = blockIdx.x;
        beg = bx * cfg.items_q + min(bx, cfg.items_r);
        end = beg + cfg.items_q + (bx < cfg.items_r ? 1 : 0);
    }
    if (beg >= end) return;
    // Warp w starts with item beg + w; every further item is claimed from this counter when a warp has consumed its
    // stage, so a warp that meets slower memory channels takes fewer items instead of holding the CTA back.
    int* s_next = reinterpret_cast<int*>(smem + 260);
    if (tid == 0) *s_next = beg + S;  // published by the barriers below
    uint8_t* my_stage = s_stage + static_cast<size_t>(warp) * cfg.stage_bytes;
    const uint32_t w_r0 = smem_u32(my_stage) + g * 128;
    const wf_problem* const h0 = reinterpret_cast<const wf_problem*>(s_hdr);
    const wf_problem* const h1 = reinterpret_cast<const wf_problem*>(s_hdr + HDR_STRIDE);
    int hdr_pi0 = -1, hdr_pi1 = -1;  // the problems whose heads the two slots hold

    // cursor of the item whose first K segment is in flight in this warp's stage (>= end: none)
    ItemCursor nx;
    int nx_item = warp < S ? beg + warp : end;
    unsigned loads = 0;  // completed + pending requests of this warp (parity of the wait)
    // head of problem pi: a cached copy if there is one, else the descriptor in global memory
    auto head_of = [&](int pi) -> const wf_problem* { return pi == hdr_pi0 ? h0 : (pi == hdr_pi1 ? h1 : &probs[pi]); };
    auto issue_first = [&](bool from_param) {
        if (nx_item < end) {
            int local;
            nx.pi = locate_problem(probs, cfg.P, nx_item, s_ib, cfg.ib_cap, local, uni);
            const wf_problem* h = from_param ? &single : head_of(nx.pi);
            nx.row_items = h->_row_items;
            nx.chunks = h->_chunks;
            nx.chunk = local / nx.row_items;
            nx.ritem = local % nx.row_items;
            if (lane == 0) {
                mbar_expect_tx(&full[warp], segment_bytes(h, 0));
                issue_segment(h, &probs[nx.pi], nx.ritem * 16, 0, my_stage, &full[warp]);
            }
        }
    };
    // Two activation buffers: the first two passes of the CTA's range are quantized up front, so that a CTA
    // whose range crosses from one problem into the next does not stop streaming there.  Later passes (rare:
    // problems much smaller than a CTA's share) reuse the buffers behind a CTA-wide barrier.
    const int act_bytes = cfg.KBmax * cfg.MTA * TOK_STRIDE;
    const int nbuf = cfg.nbuf;
    const bool early = cfg.x_early != 0;  // equal problems whose x lie at a constant stride: x is found without a head
    int pre_chunk0 = 0, pre_chunk1 = 0, pre_end0 = end, pre_end1 = end, npre = 1;
    int local0, local1 = 0;
    hdr_pi0 = locate_problem(probs, cfg.P, beg, s_ib, cfg.ib_cap, local0, uni);
    uint32_t hw0 = 0, hw1 = 0;  // head words on their way from global memory (equal problems)
    if (uni > 0) {
        const int ri = single._row_items;  // the geometry of the passes follows from the parameter copy
        pre_chunk0 = local0 / ri;
        pre_end0 = min(end, beg - local0 + (pre_chunk0 + 1) * ri);
        if (nbuf > 1 && pre_end0 < end) {
            hdr_pi1 = locate_problem(probs, cfg.P, pre_end0, s_ib, cfg.ib_cap, local1, uni);
            pre_chunk1 = local1 / ri;
            pre_end1 = min(end, pre_end0 - local1 + (pre_chunk1 + 1) * ri);
            npre = 2;
        }
        if (!(cfg.x_ready && early)) issue_first(true);
        if (tid < HDR_WORDS) hw0 = reinterpret_cast<const uint32_t*>(&probs[hdr_pi0])[tid];
        if (npre > 1 && tid >= 64 && tid < 64 + HDR_WORDS) hw1 = reinterpret_cast<const uint32_t*>(&probs[hdr_pi1])[tid - 64];
    } else {
        fill_header(s_hdr, &probs[hdr_pi0], tid);
        __syncthreads();
        pre_chunk0 = local0 / h0->_row_items;
        pre_end0 = min(end, beg - local0 + (pre_chunk0 + 1) * h0->_row_items);
        if (nbuf > 1 && pre_end0 < end) {
            hdr_pi1 = locate_problem(probs, cfg.P, pre_end0, s_ib, cfg.ib_cap, local1, uni);
            fill_header(s_hdr + HDR_STRIDE, &probs[hdr_pi1], tid - 64);
            __syncthreads();
            pre_chunk1 = local1 / h1->_row_items;
            pre_end1 = min(end, pre_end0 - local1 + (pre_chunk1 + 1) * h1->_row_items);
            npre = 2;
        }
        if (!cfg.x_ready) issue_first(false);
    }
    auto store_heads = [&]() {
        if (tid < HDR_WORDS) reinterpret_cast<uint32_t*>(s_hdr)[tid] = hw0;
        if (npre > 1 && tid >= 64 && tid < 64 + HDR_WORDS) reinterpret_cast<uint32_t*>(s_hdr + HDR_STRIDE)[tid - 64] = hw1;
    };
    if (cfg.prefetch) issue_l2_prefetch(probs, cfg.P, tid, STREAM_THREADS);  // behind this CTA's own first requests
    // The weights never depend on the previous kernel, x normally does: request weights, wait, read x.  Where the
    // caller states that x is ready, the reads of x are started first and only the stores wait for the previous kernel.
    if (!cfg.x_ready) asm volatile("griddepcontrol.wait;\n" ::: "memory");
    uint8_t* const s_xchg = smem + XCHG_SMEM_OFF;
    if (cfg.xchg) xchg_fetch_async(cfg.xchg, s_xchg, tid);  // used at the end (a pushing launch always waits here: see run_group)
    if (uni > 0 && !early) {  // x is found through the heads
        store_heads();
        __syncthreads();
    }
    const wf_problem& q0 = early ? single : *h0;  // scalar fields for the first two phases
    const wf_problem& q1 = early ? single : *h1;
    const void* x0 = early ? static_cast<const void*>(static_cast<const char*>(cfg.x_base) + hdr_pi0 * cfg.x_stride) : h0->x;
    const float* xs0 = early ? nullptr : h0->x_scale;
    const void* x1 = nullptr;
    const float* xs1 = nullptr;
    if (npre > 1) {
        x1 = early ? static_cast<const void*>(static_cast<const char*>(cfg.x_base) + hdr_pi1 * cfg.x_stride) : h1->x;
        xs1 = early ? nullptr : h1->x_scale;
    }
    const int m00 = pre_chunk0 * cfg.MTA, mv0 = min(cfg.MTA, single.M - m00);  // M of the first problem: see below
    const int m01 = pre_chunk1 * cfg.MTA;
    XCache<XDT> xcache0, xcache1;
    const int mvalid0 = uni > 0 ? mv0 : min(cfg.MTA, h0->M - m00);
    const int mvalid1 = npre > 1 ? min(cfg.MTA, (uni > 0 ? single.M : h1->M) - m01) : 0;
    // fused input modes: the CTA that owns the first row item of a (problem, token pass) writes the residual stream
    const bool wh0 = !early && uni == 0 && h0->h_out != nullptr && (local0 % h0->_row_items) == 0;
    const bool wh1 = npre > 1 && !early && uni == 0 && h1->h_out != nullptr && (local1 % h1->_row_items) == 0;
    quantize_phase<XDT, STREAM_THREADS, Q_ISSUE>(q0, x0, xs0, cfg.MTA, m00, mvalid0, s_act, s_inv, s_rowsum, s_maxbits, xcache0, s_ss, wh0);
    if (npre > 1)
        quantize_phase<XDT, STREAM_THREADS, Q_ISSUE>(q1, x1, xs1, cfg.MTA, m01, mvalid1, s_act + act_bytes, s_inv + MT, s_rowsum + MT,
                                                     s_maxbits + MT, xcache1, s_ss + MT * 16, wh1);
    if (cfg.x_ready && (early || uni == 0)) issue_first(early);  // behind the reads of x
    if (early) store_heads();  // published by the barrier that opens the next phase
    quantize_phase<XDT, STREAM_THREADS, Q_ABSMAX>(q0, x0, xs0, cfg.MTA, m00, mvalid0, s_act, s_inv, s_rowsum, s_maxbits, xcache0, s_ss, wh0);
    if (npre > 1)
        quantize_phase<XDT, STREAM_THREADS, Q_ABSMAX>(q1, x1, xs1, cfg.MTA, m01, mvalid1, s_act + act_bytes, s_inv + MT, s_rowsum + MT,
                                                      s_maxbits + MT, xcache1, s_ss + MT * 16, wh1);
    quantize_phase<XDT, STREAM_THREADS, Q_EMIT>(q0, x0, xs0, cfg.MTA, m00, mvalid0, s_act, s_inv, s_rowsum, s_maxbits, xcache0, s_ss, wh0);
    if (npre > 1)
        quantize_phase<XDT, STREAM_THREADS, Q_EMIT>(q1, x1, xs1, cfg.MTA, m01, mvalid1, s_act + act_bytes, s_inv + MT, s_rowsum + MT,
                                                    s_maxbits + MT, xcache1, s_ss + MT * 16, wh1);
    bool may_store = !cfg.x_ready;  // the previous kernel has been waited for

    int it = beg;
    for (int seg = 0; it < end; ++seg) {
        const int buf = seg % nbuf;
        uint8_t* const slot = s_hdr + buf * HDR_STRIDE;
        const wf_problem& p = *reinterpret_cast<const wf_problem*>(slot);
        int pi, chunk, seg_end;
        if (seg < npre) {
            pi = seg == 0 ? hdr_pi0 : hdr_pi1;
            chunk = seg == 0 ? pre_chunk0 : pre_chunk1;
            seg_end = seg == 0 ? pre_end0 : pre_end1;
        } else {
            consumer_sync<STREAM_THREADS>();  // every warp is done with the pass that used this buffer and this head
            int local;
            pi = locate_problem(probs, cfg.P, it, s_ib, cfg.ib_cap, local, uni);
            fill_header(slot, &probs[pi], tid);
            if (buf == 0) hdr_pi0 = pi; else hdr_pi1 = pi;
            consumer_sync<STREAM_THREADS>();
            chunk = local / p._row_items;
            seg_end = min(end, it - local + (chunk + 1) * p._row_items);
            const int m0q = chunk * cfg.MTA;
            quantize_tokens<XDT, STREAM_THREADS>(p, cfg.MTA, m0q, min(cfg.MTA, p.M - m0q), s_act + buf * act_bytes, s_inv + buf * MT,
                                                 s_rowsum + buf * MT, s_maxbits + buf * MT, s_ss + buf * MT * 16,
                                                 p.h_out != nullptr && (local % p._row_items) == 0);
        }
        const int m0 = chunk * cfg.MTA, m_valid = min(cfg.MTA, p.M - m0);
        const int ritem = it - first_item(probs, pi, s_ib, cfg.ib_cap, uni) - chunk * p._row_items;
        const wf_problem* const gp = &probs[pi];
        const uint32_t act0 = smem_u32(s_act + buf * act_bytes);
        const float* const inv_p = s_inv + buf * MT;
        const int* const rowsum_p = s_rowsum + buf * MT;
        const int KB = (p.K + 511) >> 9, kb_seg = p._kb_seg, ksegs = p._ksegs;
        const float s_w = p.w_scale ? __ldg(p.w_scale) : p.w_scale_host;
        void* const y = p.y;
        const void* const bias = p.bias;
        int32_t* const acc_out = p.acc_out;
        const int64_t ldy = p.ldy;
        const int N = p.N, y_dtype = p.y_dtype, bias_dtype = p.bias_dtype;
        {
            while (nx_item < seg_end) {  // this warp's items of the pass
                const int j = nx_item;
                int acc[NT][FOURACC ? 4 : 1][4];
#pragma unroll
                for (int a = 0; a < NT; ++a)
#pragma unroll
                    for (int b = 0; b < (FOURACC ? 4 : 1); ++b)
#pragma unroll
                        for (int c = 0; c < 4; ++c) acc[a][b][c] = 0;
                const int my_row = (ritem + (j - it)) * 16;
                // K arrives in segments through this warp's one stage; after each the warp requests what it needs next
                for (int ks = 0; ks < ksegs; ++ks) {
                    mbar_wait(&full[warp], loads & 1, poisoned);
                    ++loads;
                    const int kb0 = ks * kb_seg, kbn = min(KB - kb0, kb_seg);
#pragma unroll 1
                    for (int i = 0; i < kbn; ++i)
                        compute_unit<NT, FOURACC>(w_r0 + i * TILE_BYTES, w_r0 + i * TILE_BYTES + 1024,
                                                  act0 + (kb0 + i) * cfg.MTA * TOK_STRIDE, m_valid, g, t, acc);
                    __syncwarp();  // the stage has been read
                    if (ks + 1 < ksegs) {
                        if (lane == 0) {
                            asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
                            mbar_expect_tx(&full[warp], segment_bytes(&p, ks + 1));
                            issue_segment(&p, gp, my_row, ks + 1, my_stage, &full[warp]);
                        }
                    } else {
                        int claimed = 0;  // this warp's next item (it may belong to a later pass)
                        if (lane == 0) claimed = atomicAdd(s_next, 1);
                        claimed = __shfl_sync(0xffffffffu, claimed, 0);
                        const int step = claimed - nx_item;
                        nx_item = claimed < end ? claimed : end;
                        if (nx_item < end) {
                            nx.ritem += step;
                            while (nx.ritem >= nx.row_items) {
                                nx.ritem -= nx.row_items;
                                if (++nx.chunk == nx.chunks) {
                                    nx.chunk = 0;
                                    ++nx.pi;  // nx_item < end: the problem exists
                                    const wf_problem* h = head_of(nx.pi);
                                    nx.row_items = h->_row_items;
                                    nx.chunks = h->_chunks;
                                }
                            }
                            if (lane == 0) {
                                const wf_problem* h = head_of(nx.pi);
                                asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
                                mbar_expect_tx(&full[warp], segment_bytes(h, 0));
                                issue_segment(h, &probs[nx.pi], nx.ritem * 16, 0, my_stage, &full[warp]);
                            }
                        }
                    }
                }
                if (!may_store) {  // y may still be in use by the previous kernel
                    asm volatile("griddepcontrol.wait;\n" ::: "memory");
                    may_store = true;
                }
                // epilogue straight from the accumulators: lane holds rows g, g+8 x tokens 2t, 2t+1 of every token tile
                const int row_a = my_row + g, row_b = row_a + 8;
#pragma unroll
                for (int nt = 0; nt < NT; ++nt) {
#pragma unroll
                    for (int c = 0; c < 4; ++c) {
                        int v;
                        if constexpr (FOURACC)
                            v = acc[nt][0][c] + (acc[nt][1][c] >> 2) + (acc[nt][2][c] >> 4) + (acc[nt][3][c] >> 6);
                        else
                            v = acc[nt][0][c];
                        const int tok = nt * 8 + 2 * t + (c & 1);
                        const int nrow = (c & 2) ? row_b : row_a;
                        if (tok < m_valid && nrow < N) {
                            const int a = v - rowsum_p[tok];
                            float out = rescale(a, inv_p[tok], s_w);
                            if (bias) out = __fadd_rn(out, load1_rt(bias, bias_dtype, nrow));
                            const int64_t m = m0 + tok;
                            store1_rt(y, y_dtype, m * ldy + nrow, out);
                            if (acc_out) acc_out[m * N + nrow] = a;
                        }
                    }
                }
            }
        }
        it = seg_end;
    }
    // a kernel that follows with a programmatic dependency relies on this grid having waited for its own predecessor
    if (!may_store) asm volatile("griddepcontrol.wait;\n" ::: "memory");
    if (cfg.xchg) {
        xchg_fetch_wait(tid);
        __syncthreads();  // every warp's outputs are written
        xchg_push_items<STREAM_THREADS>(cfg, probs, beg, end, 16, s_ib, uni, tid, s_xchg);
    }
}

// ------------------------------------------------------------------ host side
struct GroupPlan {
    int NT, RI, KBmax, MTA, stages, stage_bytes, act_off, stage_off, total_items, grid, decoupled, cpp, nbuf;
    size_t smem;
};

constexpr size_t SMEM_MAX = 227 * 1024;
constexpr size_t SMEM_STREAM_MAX = 113 * 1024;  // two streaming CTAs per SM

static long long count_items16(const wf_problem* probs, int P, int MT) {
    long long t = 0;
    for (int i = 0; i < P; ++i) t += static_cast<long long>((probs[i].N + 15) / 16) * ((probs[i].M + MT - 1) / MT);
    return t;
}

constexpr int IB_CAP = 1024;  // problems whose first item index is cached in shared memory

static size_t ss_offset(int NT, int RI) {  // the norm's partial sums follow the per-token constants and the reduction tiles
    const int MT = NT * 8;
    return (384 + static_cast<size_t>(MT) * 24 + 2u * RI * 16 * MT * 4 + 15) / 16 * 16;
}
static size_t fixed_bytes(int NT, int RI) {
    const int MT = NT * 8;
    size_t b = ss_offset(NT, RI) + 2u * MT * 16 * 4;
    return (b + 127) / 128 * 128 + IB_CAP * 4 + 384;  // + table of first items + two descriptor heads
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(p);
    }
    return fn;
}

constexpr int KB_SEG_MAX = 7;  // 512-weight blocks per streamed K segment: 14 KB per 16-row tile

static void k_segments(int K, int& kb_seg, int& ksegs) {
    const int KB = (K + 511) / 512;
    ksegs = (KB + KB_SEG_MAX - 1) / KB_SEG_MAX;
    kb_seg = (KB + ksegs - 1) / ksegs;
    ksegs = (KB + kb_seg - 1) / kb_seg;
}

// TMA descriptors of the packed weights of one problem.  Main: the full 128-byte column blocks as a 3-D tensor
// [block][row][128 bytes] with a box of [_kb_seg blocks][16 rows][128], so that one request lands a K segment of a
// row tile in a stage as consecutive 2 KB tiles; Last: the same view with the shorter box of the last segment;
// Tail: the last, partial column block as a 2-D tensor whose missing bytes are filled with zeros.  When the 3-D
// view is refused, the plain 2-D view [row][K/4 bytes] is used with one request per column block.
static int encode_maps(wf_problem& q) {
    EncodeTiledFn enc = encode_fn();
    if (!enc) return fail(WF_E_DEVICE, "cuTensorMapEncodeTiled is not available in this driver");
    const cuuint64_t rowbytes = static_cast<cuuint64_t>(q.K) / 4;
    const int kbf = static_cast<int>(rowbytes / 128), tail = static_cast<int>(rowbytes % 128);
    int kb_seg, ksegs;
    k_segments(q.K, kb_seg, ksegs);
    q._kb_seg = kb_seg;
    q._ksegs = ksegs;
    const cuuint32_t ones[3] = {1, 1, 1};
    void* base = const_cast<uint8_t*>(q.codes);
    auto enc3 = [&](uint64_t* out, int box_blocks) {
        const cuuint64_t dims[3] = {128, static_cast<cuuint64_t>(q.N), static_cast<cuuint64_t>(kbf)};
        const cuuint64_t strides[2] = {rowbytes, 128};
        const cuuint32_t box[3] = {128, 16, static_cast<cuuint32_t>(box_blocks)};
        return enc(reinterpret_cast<CUtensorMap*>(out), CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, base, dims, strides, box, ones,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    };
    CUresult r = CUDA_SUCCESS;
    if (kbf > 0) {
        // a segment holds either _kb_seg full blocks (main box) or, the last one, fewer (its own box)
        if (kbf >= kb_seg) r = enc3(q._tmap_main, kb_seg);
        const int last_full = kbf - (ksegs - 1) * kb_seg;  // full blocks of the last segment (may be <= 0)
        if (r == CUDA_SUCCESS && last_full > 0 && last_full != kb_seg) r = enc3(q._tmap_last, last_full);
    }
    if (kbf > 0 && r == CUDA_SUCCESS) {
        q._kb_full = kbf;
        q._tail_bytes = tail;
        if (tail) {
            const cuuint64_t dims[2] = {static_cast<cuuint64_t>(tail), static_cast<cuuint64_t>(q.N)};
            const cuuint64_t strides[1] = {rowbytes};
            const cuuint32_t box[2] = {128, 16};
            r = enc(reinterpret_cast<CUtensorMap*>(q._tmap_tail), CU_TENSOR_MAP_DATA_TYPE_UINT8, 2,
                    static_cast<uint8_t*>(base) + static_cast<size_t>(kbf) * 128, dims, strides, box, ones,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
            if (r != CUDA_SUCCESS) return fail(WF_E_DEVICE, "cuTensorMapEncodeTiled (tail block) failed with %d", (int)r);
        }
        return WF_OK;
    }
    // plain 2-D view
    const cuuint64_t dims[2] = {rowbytes, static_cast<cuuint64_t>(q.N)};
    const cuuint64_t strides[1] = {rowbytes};
    const cuuint32_t box[2] = {128, 16};
    r = enc(reinterpret_cast<CUtensorMap*>(q._tmap_tail), CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, base, dims, strides, box, ones,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(WF_E_DEVICE, "cuTensorMapEncodeTiled failed with %d", (int)r);
    q._kb_full = 0;
    q._tail_bytes = static_cast<int>(rowbytes);
    return WF_OK;
}

// All problems read the same tokens in one pass (q/k/v, gate/up, or a single problem): one quantization serves them all.
static bool shares_x(const wf_problem* probs, int P, int MTA) {
    if (probs[0].M > MTA || probs[0].M > 8) return false;  // measured with up to 8 tokens (one token tile)
    for (int i = 1; i < P; ++i)
        if (probs[i].x != probs[0].x || probs[i].x_scale != probs[0].x_scale || probs[i].ldx != probs[0].ldx || probs[i].M != probs[0].M ||
            probs[i].K != probs[0].K || probs[i].layout != probs[0].layout || probs[i].eps != probs[0].eps ||
            probs[i].x_mode != probs[0].x_mode || probs[i].x2 != probs[0].x2 || probs[i].norm_w != probs[0].norm_w ||
            probs[i].norm_eps != probs[0].norm_eps)
            return false;
    return true;
}

// Chooses the token tile, the item size and the ring depth for a group, and fills the item fields.
static int plan_group(wf_problem* probs, int P, GroupPlan& g, bool write_fields) {
    int Kmax = 0, Mmax = 0;
    for (int i = 0; i < P; ++i) {
        Kmax = probs[i].K > Kmax ? probs[i].K : Kmax;
        Mmax = probs[i].M > Mmax ? probs[i].M : Mmax;
    }
    const int sms = num_sms();
    g.KBmax = (Kmax + 511) / 512;
    const int pitch = g.KBmax * 128;  // stage bytes per weight row
    // token tile: as many tokens as fit beside three 16-row stages
    int NT = Mmax <= 8 ? 1 : (Mmax <= 16 ? 2 : (Mmax <= 32 ? 4 : 8));
    for (;; NT >>= 1) {
        const int mta = Mmax < NT * 8 ? Mmax : NT * 8;
        const size_t need = fixed_bytes(NT, 1) + static_cast<size_t>(g.KBmax) * mta * TOK_STRIDE + 3u * 16 * pitch;
        if (need <= SMEM_MAX || NT == 1) break;
    }
    g.NT = NT;
    const int MT = NT * 8;
    g.MTA = Mmax < MT ? Mmax : MT;
    // very large K: fewer tokens per pass, until the activations fit beside two 16-row stages
    while (g.MTA > 1 && fixed_bytes(NT, 1) + static_cast<size_t>(g.KBmax) * g.MTA * TOK_STRIDE + 2u * 16 * pitch > SMEM_MAX)
        g.MTA = (g.MTA + 1) / 2;
    const size_t act = (static_cast<size_t>(g.KBmax) * g.MTA * TOK_STRIDE + 127) / 128 * 128;
    // Enough 16-row items to give every consumer warp of every SM several of them: the warps work on their
    // own items.  Otherwise (a single small layer) the 16 warps of a CTA share each item and split K.
    // streaming form: a stage holds one K segment of a 16-row tile
    int seg_max = 1;
    for (int i = 0; i < P; ++i) {
        int kb_seg, ksegs;
        k_segments(probs[i].K, kb_seg, ksegs);
        seg_max = kb_seg > seg_max ? kb_seg : seg_max;
    }
    const size_t seg_stage = static_cast<size_t>(seg_max) * TILE_BYTES;
    g.decoupled = count_items16(probs, P, g.MTA) >= 32LL * sms && fixed_bytes(NT, 1) + act + 4u * seg_stage <= SMEM_STREAM_MAX;
    // CTA ranges aligned to the problems (see g.cpp below) with all tokens in one pass: a CTA never meets a second pass
    bool one_pass = false;
    if (g.decoupled && P <= 2 * sms && Mmax <= g.MTA) {
        const int c = 2 * sms / P;
        one_pass = c * P * 10 >= 2 * sms * 9;
    }
    g.nbuf = (g.decoupled && !one_pass && fixed_bytes(NT, 1) + 2 * act + 6u * seg_stage <= SMEM_STREAM_MAX) ? 2 : 1;
    // item size: about 32 KB per stage, smaller while there are too few items to keep every SM busy
    int RI = g.decoupled ? 1 : 8;
    while (RI > 1 && 16 * RI * pitch > 32 * 1024) RI >>= 1;
    auto count_items = [&](int ri) {
        long long t = 0;
        for (int i = 0; i < P; ++i)
            t += static_cast<long long>((probs[i].N + 16 * ri - 1) / (16 * ri)) * ((probs[i].M + g.MTA - 1) / g.MTA);
        return t;
    };
    while (RI > 1 && count_items(RI) < 4LL * sms) RI >>= 1;
    while (RI > 1 && fixed_bytes(NT, RI) + act + 2u * 16 * RI * pitch > SMEM_MAX) RI >>= 1;
    // several 16-row items per CTA on shared tokens: every warp takes whole items (see the kernel), items of 16 rows
    if (!g.decoupled && shares_x(probs, P, g.MTA) && count_items(1) >= 3LL * sms) RI = 1;
    g.RI = RI;
    g.stage_bytes = g.decoupled ? static_cast<int>(seg_stage) : 16 * RI * pitch;
    g.act_off = static_cast<int>(fixed_bytes(NT, RI));
    g.stage_off = g.act_off + static_cast<int>(g.nbuf * act);
    if (static_cast<size_t>(g.stage_off) + 2u * g.stage_bytes > SMEM_MAX)
        return fail(WF_E_LIMIT, "wf_bitlinear_decode: K=%d needs more shared memory than one SM has", Kmax);
    const long long total = count_items(RI);
    if (total > 0x7fffffffLL) return fail(WF_E_LIMIT, "wf_bitlinear_decode: too many work items");
    g.total_items = static_cast<int>(total);
    g.grid = g.decoupled ? 2 * sms : (g.total_items < sms ? g.total_items : sms);  // one CTA of the shared form per SM: no second wave
    g.cpp = 0;
    if (g.decoupled && P <= g.grid) {
        const int cpp = g.grid / P;
        if (cpp * P * 10 >= g.grid * 9) g.cpp = cpp;  // at most a tenth of the CTAs left without work
    }
    const int per_cta = (g.total_items + g.grid - 1) / g.grid;
    int stages = static_cast<int>(((g.decoupled ? SMEM_STREAM_MAX : SMEM_MAX) - g.stage_off) / g.stage_bytes);
    if (stages > MAX_STAGES) stages = MAX_STAGES;
    if (!g.decoupled && stages > per_cta + 1) stages = per_cta + 1 > 2 ? per_cta + 1 : 2;
    if (g.decoupled && stages > SW) stages = SW;  // one owning warp per stage
    g.stages = stages;
    g.smem = static_cast<size_t>(g.stage_off) + static_cast<size_t>(stages) * g.stage_bytes;
    if (write_fields) {
        int begin = 0;
        for (int i = 0; i < P; ++i) {
            probs[i]._item_begin = begin;
            probs[i]._row_items = (probs[i].N + 16 * RI - 1) / (16 * RI);
            probs[i]._chunks = (probs[i].M + g.MTA - 1) / g.MTA;
            begin += probs[i]._row_items * probs[i]._chunks;
            if (int rc = encode_maps(probs[i])) return rc;
        }
    }
    return WF_OK;
}

template <int XDT, int NT, bool FOURACC>
static int launch_decode(const wf_problem* dev, const wf_problem& single, const DecodeCfg& cfg, const GroupPlan& g, unsigned flags,
                         cudaStream_t st) {
    auto kern = g.decoupled ? decode_stream_kernel<XDT, NT, FOURACC> : decode_kernel<XDT, NT, FOURACC>;
    static PerDeviceOnce configured[2];  // per instantiation and kernel form; the attribute is a per-device setting
    const int dev_now = current_device();
    if (configured[g.decoupled].needs(dev_now)) {
        WF_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(SMEM_MAX)));
        configured[g.decoupled].mark(dev_now);
    }
    cudaLaunchConfig_t lc = {};
    lc.gridDim = dim3(g.grid);
    lc.blockDim = dim3(g.decoupled ? STREAM_THREADS : DEC_THREADS);
    lc.dynamicSmemBytes = g.smem;
    lc.stream = st;
    cudaLaunchAttribute attr[1];
    if (flags & WF_FLAG_PDL) {
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = 1;
        lc.attrs = attr;
        lc.numAttrs = 1;
    }
    WF_CUDA(cudaLaunchKernelEx(&lc, kern, dev, single, cfg));
    return WF_OK;
}

template <int XDT>
static int dispatch_nt(const wf_problem* dev, const wf_problem& single, const DecodeCfg& cfg, const GroupPlan& g, unsigned flags,
                       cudaStream_t st) {
    switch (g.NT) {
        case 1: return launch_decode<XDT, 1, true>(dev, single, cfg, g, flags, st);
        case 2: return launch_decode<XDT, 2, true>(dev, single, cfg, g, flags, st);
        case 4: return launch_decode<XDT, 4, false>(dev, single, cfg, g, flags, st);
        default: return launch_decode<XDT, 8, false>(dev, single, cfg, g, flags, st);
    }
}

static int check_problem(const char* who, const wf_problem& q);

static int run_group(const char* who, const wf_problem* dev, wf_problem* host, int P, bool planned, unsigned flags, void* stream) {
    for (int i = 0; i < P; ++i) {
        if (int rc = check_problem(who, host[i])) return rc;
        WF_REQUIRE(host[i].x_dtype == host[0].x_dtype, "%s: all problems of a group must share x_dtype", who);
    }
    if (int rc = require_device()) return rc;
    GroupPlan g;
    if (planned) {
        // the caller's copy on the device was planned earlier: recompute and compare
        if (int rc = plan_group(host, P, g, false)) return rc;
        int begin = 0;
        for (int i = 0; i < P; ++i) {
            const int ri = (host[i].N + 16 * g.RI - 1) / (16 * g.RI), ch = (host[i].M + g.MTA - 1) / g.MTA;
            int kb_seg, ksegs;
            k_segments(host[i].K, kb_seg, ksegs);
            WF_REQUIRE(host[i]._item_begin == begin && host[i]._row_items == ri && host[i]._chunks == ch &&
                           host[i]._kb_seg == kb_seg && host[i]._ksegs == ksegs,
                       "%s: problem %d was not prepared by wf_bitlinear_decode_plan (or was changed afterwards)", who, i);
            begin += ri * ch;
        }
    } else {
        if (int rc = plan_group(host, P, g, true)) return rc;
    }
    DecodeCfg cfg;
    cfg.P = P; cfg.total_items = g.total_items; cfg.RI = g.RI; cfg.KBmax = g.KBmax; cfg.MTA = g.MTA; cfg.stages = g.stages;
    cfg.stage_bytes = g.stage_bytes; cfg.act_off = g.act_off; cfg.stage_off = g.stage_off; cfg.decoupled = g.decoupled; cfg.cpp = g.cpp; cfg.nbuf = g.nbuf;
    cfg.ib_cap = P < IB_CAP ? P : IB_CAP; cfg.ib_off = g.act_off - IB_CAP * 4 - 384; cfg.hdr_off = g.act_off - 384;
    cfg.ss_off = static_cast<int>(ss_offset(g.NT, g.RI));
    cfg.xchg = nullptr;
    for (int i = 0; i < P; ++i) {
        if (!host[i].xchg) continue;
        if (cfg.xchg) return fail(WF_E_ARG, "%s: one problem of a launch may push to an exchange (its output fills the exchange's slot)", who);
        cfg.xchg = host[i].xchg;
    }
    cfg.prefetch = 0;
    if (P <= 8)
        for (int i = 0; i < P; ++i) cfg.prefetch |= (host[i].prefetch != nullptr && host[i].prefetch_bytes > 0) ? 1 : 0;
    cfg.x_ready = ((flags & WF_FLAG_X_READY) && !cfg.xchg) ? 1 : 0;  // a pushing launch reads the exchange's step after its predecessors
    cfg.wide = (!g.decoupled && g.RI == 1 && g.total_items >= 3LL * g.grid && shares_x(host, P, g.MTA)) ? 1 : 0;
    cfg.items_q = g.total_items / g.grid; cfg.items_r = g.total_items % g.grid;
    cfg.uniform_items = 0;
    if (g.decoupled) {
        bool same = true;
        for (int i = 1; i < P && same; ++i)
            same = host[i].M == host[0].M && host[i].N == host[0].N && host[i].K == host[0].K && host[i].layout == host[0].layout;
        if (same) cfg.uniform_items = host[0]._row_items * host[0]._chunks;
    }
    cfg.x_early = 0; cfg.x_base = host[0].x; cfg.x_stride = 0;
    if (cfg.uniform_items > 0) {
        const char* b0 = static_cast<const char*>(host[0].x);
        const long long dx = P > 1 ? static_cast<const char*>(host[1].x) - b0 : 0;
        bool ok = host[0].x_scale == nullptr && host[0].ldx == host[P > 1 ? 1 : 0].ldx;
        for (int i = 0; i < P && ok; ++i) ok = host[i].x_mode == WF_X_PLAIN;  // fused inputs are found through the heads
        for (int i = 1; i < P && ok; ++i)
            ok = host[i].x_scale == nullptr && host[i].ldx == host[0].ldx && host[i].eps == host[0].eps &&
                 static_cast<const char*>(host[i].x) - b0 == dx * i;
        if (ok) { cfg.x_early = 1; cfg.x_stride = dx; }
    }
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    // A group of one problem travels as a kernel parameter, like a single launch: its fields and tensor maps are then read
    // without a round trip to global memory at the kernel's entry.
    if (P == 1) dev = nullptr;
    switch (host[0].x_dtype) {
        case WF_F32: return dispatch_nt<WF_F32>(dev, host[0], cfg, g, flags, st);
        case WF_BF16: return dispatch_nt<WF_BF16>(dev, host[0], cfg, g, flags, st);
        case WF_F16: return dispatch_nt<WF_F16>(dev, host[0], cfg, g, flags, st);
        default: return dispatch_nt<WF_I8>(dev, host[0], cfg, g, flags, st);
    }
}

}  // namespace wf

using namespace wf;

// Shared argument validation of the contraction entry points.
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

static int wf::check_problem(const char* who, const wf_problem& q) {
    if (int rc = wf_check_linear_args(who, q.x, q.x_dtype, q.ldx, q.x_scale, q.codes, q.layout, q.bias, q.bias_dtype, q.y, q.y_dtype,
                                      q.ldy, q.M, q.N, q.K))
        return rc;
    WF_REQUIRE(q.x_mode >= WF_X_PLAIN && q.x_mode <= WF_X_NORM, "%s: unknown x_mode %d", who, q.x_mode);
    WF_REQUIRE(q.prefetch_bytes >= 0 && q.prefetch_bytes % 16 == 0 && (reinterpret_cast<uintptr_t>(q.prefetch) & 15) == 0,
               "%s: the prefetch range must be 16-byte aligned and a multiple of 16 bytes", who);
    if (q.xchg)
        WF_REQUIRE((q.y_dtype == WF_BF16 || q.y_dtype == WF_F16) && q.ldy == q.N && q.N % 2 == 0 && (reinterpret_cast<uintptr_t>(q.y) & 3) == 0,
                   "%s: a fused exchange needs a contiguous 16-bit output with an even number of columns", who);
    if (q.x_mode != WF_X_PLAIN) {
        WF_REQUIRE(q.x_dtype == WF_BF16, "%s: fused input modes take bf16 tensors", who);
        WF_REQUIRE(q.K % 8 == 0, "%s: fused input modes need K %% 8 == 0", who);
        auto al16 = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; };
        if (q.x_mode == WF_X_NORM)
            WF_REQUIRE(q.norm_w && al16(q.norm_w) && al16(q.x2) && al16(q.h_out), "%s: the RMSNorm input mode needs a 16-byte aligned norm_w (x2, h_out optional, aligned)", who);
        else
            WF_REQUIRE(q.x2 && al16(q.x2), "%s: the activation input modes need x2 (the `up` tensor), 16-byte aligned", who);
    }
    return WF_OK;
}

extern "C" int wf_bitlinear_decode(const void* x, int x_dtype, int64_t ldx, const float* x_scale, const uint8_t* codes,
                                   int layout, const float* w_scale, float w_scale_host, const void* bias, int bias_dtype,
                                   void* y, int y_dtype, int64_t ldy, int32_t* acc_out, int64_t M, int64_t N, int64_t K,
                                   float eps, unsigned flags, void* stream) {
    if (int rc = wf_check_linear_args("wf_bitlinear_decode", x, x_dtype, ldx, x_scale, codes, layout, bias, bias_dtype, y,
                                      y_dtype, ldy, M, N, K))
        return rc;
    wf_problem p = {};
    p.x = x; p.x_scale = x_scale; p.codes = codes; p.w_scale = w_scale; p.bias = bias; p.y = y; p.acc_out = acc_out;
    p.ldx = ldx; p.ldy = ldy; p.M = static_cast<int>(M); p.N = static_cast<int>(N); p.K = static_cast<int>(K);
    p.x_dtype = x_dtype; p.y_dtype = y_dtype; p.bias_dtype = bias_dtype; p.layout = layout;
    p.w_scale_host = w_scale_host; p.eps = eps;
    return run_group("wf_bitlinear_decode", nullptr, &p, 1, false, flags, stream);
}

extern "C" int wf_bitlinear_decode_plan(wf_problem* host_problems, int P) {
    WF_REQUIRE(host_problems && P > 0, "wf_bitlinear_decode_plan: empty group");
    for (int i = 0; i < P; ++i)
        if (int rc = check_problem("wf_bitlinear_decode_plan", host_problems[i])) return rc;
    if (int rc = require_device()) return rc;
    GroupPlan g;
    return plan_group(host_problems, P, g, true);
}

extern "C" int wf_bitlinear_decode_grouped(const wf_problem* dev_problems, const wf_problem* host_problems, int P, unsigned flags,
                                           void* stream) {
    WF_REQUIRE(dev_problems && host_problems && P > 0, "wf_bitlinear_decode_grouped: empty group");
    return run_group("wf_bitlinear_decode_grouped", dev_problems, const_cast<wf_problem*>(host_problems), P, true, flags, stream);
}

extern "C" int wf_prefill_status_fetch(int* out);
extern "C" int wf_linear_status_fetch(int* out);

extern "C" int wf_device_status(void) {
    if (int rc = require_device()) return rc;
    WF_CUDA(cudaDeviceSynchronize());
    int v = 0, v2 = 0;
    if (int rc = wf_prefill_status_fetch(&v2)) return rc;
    if (v2) return fail(v2, "a bounded wait inside the prefill kernel ran out; the outputs of that launch are invalid");
    if (int rc = wf_linear_status_fetch(&v2)) return rc;
    if (v2) return fail(v2, "a bounded wait inside the bf16 linear kernel ran out; the outputs of that launch are invalid");
    WF_CUDA(cudaMemcpyFromSymbol(&v, g_decode_status, sizeof(int)));
    if (v) {
        int zero = 0;
        WF_CUDA(cudaMemcpyToSymbol(g_decode_status, &zero, sizeof(int)));
        return fail(v, "a bounded wait inside a decode kernel ran out; the outputs of that launch are invalid");
    }
    return WF_OK;
}
