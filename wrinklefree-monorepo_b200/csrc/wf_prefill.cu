// The tensor-core contraction (prefill, and every launch with 16 or more tokens per problem): a dense int8 GEMM on
// the 5th-generation tensor cores.
//
//   acc[tok, n] = sum_k q[tok, k] * code[n, k]      (u8 codes = w + 1, s8 activations, s32 accumulate in TMEM)
//   y[tok, n]   = (float(acc - rowsum[tok]) * inv_sx[tok]) * s_w + bias[n]
//
// The weights sit on the MMA's M side: a tile is 128 weight rows x NTOK tokens (NTOK = 16 / 32 / 64 for that many
// tokens per problem, blocks of 128 beyond), and the expanded weights never touch shared memory.  Persistent CTAs (one
// per SM) walk the tiles; K advances in stages of 512:
//   * warp 0 (one lane): TMA of the PACKED weight rows (128 rows x 128 bytes, 128-byte swizzle), ring of 6 stages;
//   * warp 14 (one lane): TMA of the int8 token tile (4 swizzle atoms of NTOK x 128 bytes, the MMA's B operand);
//   * warps 2-5 / 6-9: expansion, each half takes two of a stage's four atoms; thread = weight row: 4 x ld.shared.v4, mask +
//     shift to one int8 per byte, 2 x tcgen05.st of 32 columns into a ring of tensor-memory stages;
//   * warp 1 (one lane): tcgen05.mma.cta_group::1.kind::i8 (M = 128, N = NTOK, K = 32), A operand FROM TENSOR MEMORY, sixteen
//     per stage and one commit; two accumulator buffers, so the epilogue of a tile runs under the next tile's MMAs.  The
//     forms for few tokens have two or three issuing threads (warps 1 and 19, or 1, 15 and 16), one per ring slot, each
//     with a partial accumulator of its own;
//   * warps 10-13 (and 15-18): epilogue, thread = weight row: tcgen05.ld (summing the partial accumulators), integer
//     correction, fp32 rescale, store.
// Every mbarrier wait is bounded.
#include <cuda.h>

#include "wf_common.cuh"

namespace wf {
__device__ int g_prefill_status = 0;
}
#define WF_STATUS_WORD ::wf::g_prefill_status
#include "wf_async.cuh"

int wf_check_linear_args(const char* who, const void* x, int x_dtype, int64_t ldx, const float* x_scale, const uint8_t* codes,
                         int layout, const void* bias, int bias_dtype, void* y, int y_dtype, int64_t ldy, int64_t M, int64_t N,
                         int64_t K);

namespace wf {

struct PrefillParams {
    const float* x_scale;   // [M] per-token multipliers (nullable: 1)
    const int32_t* rowsum;  // [M]
    const float* w_scale;
    float w_scale_host;
    const void* bias;
    int bias_dtype;
    void* y;
    int y_dtype;
    int64_t ldy;
    int32_t* acc_out;
    int M, N, K, layout;
    int batch;            // independent problems stacked along rows: tokens [batch*M, K], weights [batch*N, K/4]
    int w_scale_stride;   // floats between the weight scales of consecutive problems
    int tiles_m, tiles_n; // per problem: token blocks of NTOK, row blocks of 128
    int x_ready;          // the tokens, their constants and y have nothing to do with the kernels still running ahead of this
                          // one: no load or store waits for them, only the end of the grid does
};

__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory"); }
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory"); }

__device__ __forceinline__ void tc_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n" ::"r"(smem_u32(bar)) : "memory");
}

// K-major operand tile with 128-byte swizzle: rows of 128 bytes, 8-row groups 1024 bytes apart.
__device__ __forceinline__ uint64_t smem_desc_sw128(uint32_t addr) {
    uint64_t d = 0;
    d |= static_cast<uint64_t>((addr & 0x3FFFF) >> 4);  // start address
    d |= static_cast<uint64_t>(1024 >> 4) << 32;        // stride between 8-row groups
    d |= static_cast<uint64_t>(1) << 46;                // descriptor version of sm_100
    d |= static_cast<uint64_t>(2) << 61;                // SWIZZLE_128B
    return d;
}

__device__ __forceinline__ uint4 lds128p(uint32_t addr) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];\n" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
    return v;
}

// What shaped this kernel (all measured on B200): with the expanded weights staged in shared memory (32 KB written
// and read again per 128-wide K block, beside the token tile) the shared-memory port and the barrier round trips
// bounded the pipeline at about a third of the tensor rate whatever the ring depths; a blocking mbarrier wait costs
// ~260 cycles even when it succeeds at once (hence the non-blocking first test in mbar_wait); and for few tokens the
// MMA issue rate (~29 ns per instruction of K = 32 whatever N <= 64) is the floor, so a barrier round trip per
// 128-wide K block doubled the time: stages of 512 amortise it over sixteen MMAs.
constexpr int SM_BM = 128;   // weight rows per tile
constexpr int SM_BK = 128;   // K per swizzle atom (128 bytes of int8)
constexpr int SM_PK = 4;     // atoms per stage: a stage is 512 weights of every row = one 128-byte packed row segment
constexpr int SM_PS = 6;     // packed-weight stages
// Issuing threads.  One thread issues a tcgen05.mma of K = 32 every ~26 ns whatever the instruction's size; the tensor
// pipe itself needs 17 ns for N = 64 and less than 7 ns for N = 16 (measured with the A operand in tensor memory: two
// issuing threads on separate accumulators reach 13 ns per instruction, four 6.6 ns).  For few tokens per tile the
// stages are therefore shared out among several issuing threads (one per warp): thread i takes the stages that land in
// ring slot i, sixteen MMAs and one commit each, into an accumulator of its own; the epilogue adds the partial
// accumulators.  (Sharing out the four atoms of every stage instead was slower: each issuing thread then runs the whole
// per-stage bookkeeping, and a single thread's instruction stream is what limits it.)
template <int NTOK>
__host__ __device__ constexpr int sm_issuers() { return NTOK <= 16 ? 3 : (NTOK <= 64 ? 2 : 1); }
template <int NTOK>
__host__ __device__ constexpr int sm_acc_cols() { return 2 * sm_issuers<NTOK>() * NTOK <= 128 ? 128 : 256; }  // two buffers of one accumulator per issuer
constexpr int SM_A_COLS = SM_PK * SM_BK / 4;  // 128 columns of 4 int8 per stage
// token-tile stages = tensor-memory stages of expanded weights; with several issuers one ring slot per issuer
template <int NTOK>
__host__ __device__ constexpr int sm_xs() { return sm_issuers<NTOK>() > 1 ? sm_issuers<NTOK>() : (512 - sm_acc_cols<NTOK>()) / SM_A_COLS; }
constexpr int SM_P_BYTES = SM_BM * SM_PK * SM_BK / 4;  // 16 KB
constexpr int SM_THREADS = 19 * 32;
// the second issuer of the two-issuer forms is a warp of its own behind the others; the three-issuer form (16 tokens)
// uses warps that the wider forms give to their second epilogue group
template <int NTOK>
__host__ __device__ constexpr int sm_threads() { return SM_THREADS + (sm_issuers<NTOK>() == 2 ? 32 : 0); }
template <int NTOK>
constexpr size_t sm_smem() {  // more than half of an SM's shared memory: two of these CTAs never share an SM
    return 1024 + SM_PS * SM_P_BYTES + sm_xs<NTOK>() * NTOK * SM_PK * SM_BK + 2048;
}
static_assert(sm_smem<16>() > 114 * 1024 && sm_smem<64>() <= 227 * 1024 && sm_smem<128>() <= 227 * 1024, "shared memory");
static_assert(sm_acc_cols<16>() + sm_xs<16>() * SM_A_COLS <= 512 && sm_acc_cols<32>() + sm_xs<32>() * SM_A_COLS <= 512 &&
                  sm_acc_cols<64>() + sm_xs<64>() * SM_A_COLS <= 512 && sm_acc_cols<128>() + sm_xs<128>() * SM_A_COLS <= 512 &&
                  sm_xs<16>() == 3 && sm_xs<32>() == 2 && sm_xs<64>() == 2 && sm_xs<128>() == 2,
              "tensor memory");

// The four MMAs of one 128-byte swizzle atom of K in one block of PTX: A advances by 8 tensor-memory columns, B by 32
// bytes (2 in descriptor units) per step.  The issuing thread is the pipeline's critical path for few tokens, so the
// address arithmetic is kept out of the compiler's hands and the predicate is set once.
__device__ __forceinline__ void mma_i8_ts_x4(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc, uint32_t accumulate_first) {
    asm volatile(
        "{\n .reg .pred p, q;\n .reg .b32 a1, a2, a3;\n .reg .b64 b1, b2, b3;\n"
        " setp.ne.b32 p, %4, 0;\n setp.eq.b32 q, %5, %5;\n"
        " add.u32 a1, %1, 8;\n add.u32 a2, %1, 16;\n add.u32 a3, %1, 24;\n"
        " add.u64 b1, %2, 2;\n add.u64 b2, %2, 4;\n add.u64 b3, %2, 6;\n"
        " tcgen05.mma.cta_group::1.kind::i8 [%0], [%1], %2, %3, {%5, %5, %5, %5}, p;\n"
        " tcgen05.mma.cta_group::1.kind::i8 [%0], [a1], b1, %3, {%5, %5, %5, %5}, q;\n"
        " tcgen05.mma.cta_group::1.kind::i8 [%0], [a2], b2, %3, {%5, %5, %5, %5}, q;\n"
        " tcgen05.mma.cta_group::1.kind::i8 [%0], [a3], b3, %3, {%5, %5, %5, %5}, q;\n}\n" ::"r"(d_tmem),
        "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate_first), "r"(0u)
        : "memory");
}
__device__ __forceinline__ void tmem_st32(uint32_t addr, const uint32_t (&v)[32]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,"
        "%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};\n" ::"r"(addr),
        "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]), "r"(v[8]), "r"(v[9]), "r"(v[10]),
        "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15]), "r"(v[16]), "r"(v[17]), "r"(v[18]), "r"(v[19]), "r"(v[20]),
        "r"(v[21]), "r"(v[22]), "r"(v[23]), "r"(v[24]), "r"(v[25]), "r"(v[26]), "r"(v[27]), "r"(v[28]), "r"(v[29]), "r"(v[30]),
        "r"(v[31])
        : "memory");
    asm volatile("tcgen05.wait::st.sync.aligned;\n" ::: "memory");
}
__device__ __forceinline__ void tmem_st32_nowait(uint32_t addr, const uint32_t (&v)[32]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,"
        "%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};\n" ::"r"(addr),
        "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]), "r"(v[8]), "r"(v[9]), "r"(v[10]),
        "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15]), "r"(v[16]), "r"(v[17]), "r"(v[18]), "r"(v[19]), "r"(v[20]),
        "r"(v[21]), "r"(v[22]), "r"(v[23]), "r"(v[24]), "r"(v[25]), "r"(v[26]), "r"(v[27]), "r"(v[28]), "r"(v[29]), "r"(v[30]),
        "r"(v[31])
        : "memory");
}
template <int NREG>
__device__ __forceinline__ void tmem_ldn(uint32_t addr, uint32_t (&v)[NREG]);
template <>
__device__ __forceinline__ void tmem_ldn<16>(uint32_t addr, uint32_t (&v)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];\n"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]), "=r"(v[9]),
          "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
        : "r"(addr));
    asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
}

// Sixteen token columns of one weight row: integer correction, fp32 rescale, 16-bit store.  The per-token constants come
// as vectors from shared memory, the output type is decided outside the loops and the pointer runs along the token axis:
// the epilogue warps share their schedulers with the expansion warps, and at 2560-wide K a tile's epilogue (128 x 128
// outputs) used to take longer than its MMAs.
__device__ __forceinline__ void epilogue16(const uint32_t (&v)[16], const int* s_rowsum, const float* s_inv, float s_w, bool has_bias,
                                           float bias, bool is_bf16, uint16_t* yp, int64_t ldy, int valid) {
    int rs[16];
    float iv[16];
#pragma unroll
    for (int q = 0; q < 4; ++q) {
        const int4 a = *reinterpret_cast<const int4*>(s_rowsum + 4 * q);
        const float4 b = *reinterpret_cast<const float4*>(s_inv + 4 * q);
        rs[4 * q] = a.x; rs[4 * q + 1] = a.y; rs[4 * q + 2] = a.z; rs[4 * q + 3] = a.w;
        iv[4 * q] = b.x; iv[4 * q + 1] = b.y; iv[4 * q + 2] = b.z; iv[4 * q + 3] = b.w;
    }
    float o[16];
#pragma unroll
    for (int jt = 0; jt < 16; ++jt) {
        o[jt] = rescale(static_cast<int>(v[jt]) - rs[jt], iv[jt], s_w);
        if (has_bias) o[jt] = __fadd_rn(o[jt], bias);
    }
    if (valid >= 16) {
        if (is_bf16) {
#pragma unroll
            for (int jt = 0; jt < 16; ++jt, yp += ldy) *yp = __bfloat16_as_ushort(__float2bfloat16_rn(o[jt]));
        } else {
#pragma unroll
            for (int jt = 0; jt < 16; ++jt, yp += ldy) *yp = __half_as_ushort(__float2half_rn(o[jt]));
        }
    } else {
#pragma unroll
        for (int jt = 0; jt < 16; ++jt, yp += ldy)
            if (jt < valid) *yp = is_bf16 ? __bfloat16_as_ushort(__float2bfloat16_rn(o[jt])) : __half_as_ushort(__float2half_rn(o[jt]));
    }
}

template <int NTOK>
__global__ void __launch_bounds__(sm_threads<NTOK>(), 1)
    prefill_kernel(const __grid_constant__ CUtensorMap tmap_x, const __grid_constant__ CUtensorMap tmap_p, const PrefillParams p) {
    constexpr int EPI_GROUPS = NTOK >= 32 ? 2 : 1;  // epilogue warp groups; each takes NTOK / EPI_GROUPS token columns
    constexpr int EPI_COLS = NTOK / EPI_GROUPS;
    constexpr int SM_XS = sm_xs<NTOK>();
    constexpr int SM_ACC_COLS = sm_acc_cols<NTOK>();
    constexpr int NI = sm_issuers<NTOK>();   // issuing threads; with several, issuer i takes the stages of ring slot i
    constexpr int ACC_BUF = NI * NTOK;       // columns of one accumulator buffer: one partial accumulator per issuer
    static_assert(NI == 1 || NI == SM_XS, "one ring slot per issuer");
    constexpr int X_ATOM = NTOK * SM_BK;        // one 128-byte swizzle atom of the token tile
    constexpr int X_BYTES = SM_PK * X_ATOM;     // a stage: 512 values of K for every token
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
    uint8_t* p_ring = smem;                           // [SM_PS][128 rows x 128 B], 128-byte swizzle
    uint8_t* x_ring = p_ring + SM_PS * SM_P_BYTES;    // [SM_XS][SM_PK atoms][NTOK rows x 128 B], 128-byte swizzle
    uint64_t* p_full = reinterpret_cast<uint64_t*>(x_ring + SM_XS * X_BYTES);
    uint64_t* p_empty = p_full + SM_PS;
    uint64_t* a_full = p_empty + SM_PS;       // the stage's token tile has landed AND its expanded weights are in tensor memory
    uint64_t* st_free = a_full + SM_XS;       // MMA commit: token tile and tensor-memory stage may be overwritten
    uint64_t* acc_full = st_free + SM_XS;
    uint64_t* acc_empty = acc_full + 2;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
    volatile int* poisoned = reinterpret_cast<volatile int*>(tmem_slot + 1);
    // [NTOK] per-token constants of the epilogue's current token block, read as 16-byte vectors
    int* s_rowsum = reinterpret_cast<int*>((reinterpret_cast<uintptr_t>(tmem_slot + 2) + 15) & ~static_cast<uintptr_t>(15));
    float* s_inv = reinterpret_cast<float*>(s_rowsum + 128);  // [NTOK]

    // chained with a programmatic dependency: the packed weights never depend on the previous kernel (normally the
    // quantization of the tokens) and are requested at once; the token tiles and the per-token constants wait for it.
    // The kernel lets its own dependents go only when that wait is over (in the thread that loads the token tiles):
    // whatever is launched behind this grid then starts after everything ahead of it has completed, which is what a
    // following launch that waits for nothing (x_ready) relies on.  Such a launch lets its dependents go at once.
    if (p.x_ready) asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory");
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    // K is walked in stages of 512: one barrier round trip, one commit and sixteen MMAs per stage.  A last stage
    // that reaches past K is zero-filled by the TMA unit on both operands (code 0 times activation 0).
    const int stages = (p.K + SM_PK * SM_BK - 1) / (SM_PK * SM_BK);
    // tile -> (problem z, token block tb of NTOK tokens, row block rb of 128 weight rows); row blocks vary fastest, so the
    // CTAs that run side by side read the same token block
    const int tiles_per_problem = p.tiles_m * p.tiles_n;
    const int total_tiles = tiles_per_problem * p.batch;

    if (tid == 0) {
        for (int s = 0; s < SM_PS; ++s) {
            mbar_init(&p_full[s], 1);
            mbar_init(&p_empty[s], 8);
        }
        for (int s = 0; s < SM_XS; ++s) {
            mbar_init(&a_full[s], 8 + 1);  // eight expansion warps + the token tile's bytes
            mbar_init(&st_free[s], 1);
        }
        for (int a = 0; a < 2; ++a) {
            mbar_init(&acc_full[a], NI);
            mbar_init(&acc_empty[a], 4 * EPI_GROUPS);
        }
        *poisoned = 0;
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(smem_u32(tmem_slot)), "r"(512));
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::);
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    const uint32_t tmem_a = tmem_base + SM_ACC_COLS;  // SM_XS stages of SM_A_COLS columns
    // the issuing warps: warp 1, and warps 15-16 (three issuers) or warp 19 (two issuers)
    const int issuer = warp == 1 ? 0 : ((NI == 3 && warp >= 15 && warp <= 16) ? warp - 14 : ((NI == 2 && warp == 19) ? 1 : -1));

    if (warp == 0) {
        if (lane == 0) {
            // A wait that ran out ends this thread's requests (also below: token tiles, MMAs): nothing new goes into flight
            // in a CTA that has given up; the expansion and epilogue warps run on without waiting, for their barriers' sake.
            int sit = 0;
            bool live = true;
            for (int t = blockIdx.x; live && t < total_tiles; t += gridDim.x) {
                const int z = t / tiles_per_problem, rb = t % p.tiles_n;
                const int row_w = z * p.N + rb * SM_BM;
                for (int g = 0; g < stages; ++g, ++sit) {
                    const int s = sit % SM_PS;
                    if (sit >= SM_PS) live = mbar_wait(&p_empty[s], ((sit / SM_PS) - 1) & 1, poisoned);
                    if (!live) break;
                    mbar_expect_tx(&p_full[s], SM_P_BYTES);
                    tma_load_2d(p_ring + s * SM_P_BYTES, &tmap_p, g * (SM_PK * SM_BK / 4), row_w, &p_full[s]);
                }
            }
        }
    } else if (warp == 14) {
        if (lane == 0) {
            if (!p.x_ready) {
                asm volatile("griddepcontrol.wait;\n" ::: "memory");
                asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory");
            }
            int sit = 0;
            bool live = true;
            for (int t = blockIdx.x; live && t < total_tiles; t += gridDim.x) {
                const int row_x = (t / tiles_per_problem) * p.M + ((t % tiles_per_problem) / p.tiles_n) * NTOK;
                for (int g = 0; g < stages; ++g, ++sit) {
                    const int s = sit % SM_XS;
                    if (sit >= SM_XS) live = mbar_wait(&st_free[s], ((sit / SM_XS) - 1) & 1, poisoned);
                    if (!live) break;
                    mbar_expect_tx(&a_full[s], X_BYTES);
#pragma unroll
                    for (int j = 0; j < SM_PK; ++j)  // an atom that lies past K arrives as zeros
                        tma_load_2d(x_ring + s * X_BYTES + j * X_ATOM, &tmap_x, (g * SM_PK + j) * SM_BK, row_x, &a_full[s]);
                }
            }
        }
    } else if (issuer >= 0) {
        if (lane == 0) {
            // D = s32, A = unsigned 8-bit (codes, from tensor memory), B = signed 8-bit (tokens, K-major), N = NTOK, M = 128
            const uint32_t idesc = (2u << 4) | (0u << 7) | (1u << 10) | (static_cast<uint32_t>(NTOK >> 3) << 17) |
                                   (static_cast<uint32_t>(SM_BM >> 4) << 24);
            if constexpr (NI > 1) {
                // This thread's stages are those of ring slot `issuer`: operands, barriers and the accumulator column are fixed.
                uint64_t bdesc[SM_PK];
#pragma unroll
                for (int j = 0; j < SM_PK; ++j) bdesc[j] = smem_desc_sw128(smem_u32(x_ring + issuer * X_BYTES + j * X_ATOM));
                const uint32_t a_stage = tmem_a + issuer * SM_A_COLS;
                uint64_t* const my_full = &a_full[issuer];
                uint64_t* const my_free = &st_free[issuer];
                unsigned par = 0;  // parity of the next wait on my_full
                int nt = 0, sit0 = 0;
                bool live = true;
                for (int t = blockIdx.x; live && t < total_tiles; t += gridDim.x, ++nt, sit0 += stages) {
                    const int a = nt & 1;
                    const int r0 = sit0 % NI;
                    const int g0 = issuer >= r0 ? issuer - r0 : issuer - r0 + NI;  // this thread's first stage of the tile
                    if (nt >= 2) live = mbar_wait(&acc_empty[a], ((nt >> 1) - 1) & 1, poisoned);
                    if (!live) break;
                    if (g0 >= stages) {  // a tile of fewer stages than issuers: nothing of it is this thread's
                        mbar_arrive(&acc_full[a]);
                        continue;
                    }
                    tc_fence_after();
                    const uint32_t d_tmem = tmem_base + a * ACC_BUF + issuer * NTOK;
                    for (int g = g0; g < stages; g += NI) {
                        live = mbar_wait(my_full, par, poisoned);
                        if (!live) break;
                        par ^= 1;
                        tc_fence_after();
#pragma unroll
                        for (int j = 0; j < SM_PK; ++j) mma_i8_ts_x4(d_tmem, a_stage + j * 32, bdesc[j], idesc, (g != g0 || j) ? 1u : 0u);
                        tc_commit(my_free);
                    }
                    if (live) tc_commit(&acc_full[a]);
                }
            } else {
                // operand descriptors of every (stage, atom), fixed for the whole kernel
                uint64_t bdesc[SM_XS][SM_PK];
#pragma unroll
                for (int s = 0; s < SM_XS; ++s)
#pragma unroll
                    for (int j = 0; j < SM_PK; ++j) bdesc[s][j] = smem_desc_sw128(smem_u32(x_ring + s * X_BYTES + j * X_ATOM));
                int sit = 0, nt = 0;
                bool live = true;
                for (int t = blockIdx.x; live && t < total_tiles; t += gridDim.x, ++nt) {
                    const int a = nt & 1;
                    if (nt >= 2) live = mbar_wait(&acc_empty[a], ((nt >> 1) - 1) & 1, poisoned);
                    if (!live) break;
                    tc_fence_after();
                    const uint32_t d_tmem = tmem_base + a * ACC_BUF;
                    for (int g = 0; g < stages; ++g, ++sit) {
                        const int s = sit % SM_XS;
                        live = mbar_wait(&a_full[s], (sit / SM_XS) & 1, poisoned);
                        if (!live) break;
                        tc_fence_after();
                        const uint32_t a_stage = tmem_a + s * SM_A_COLS;
                        // sixteen MMAs of 32 values of K: four per swizzle atom (the ring index is resolved by a switch so
                        // that the descriptors stay in registers)
#pragma unroll
                        for (int ss = 0; ss < SM_XS; ++ss) {
                            if (ss == s) {
#pragma unroll
                                for (int j = 0; j < SM_PK; ++j)
                                    mma_i8_ts_x4(d_tmem, a_stage + j * 32, bdesc[ss][j], idesc, (g | j) ? 1u : 0u);
                            }
                        }
                        tc_commit(&st_free[s]);
                    }
                    if (live) tc_commit(&acc_full[a]);
                }
            }
        }
    } else if (warp < 10) {
        // ---- expansion: warps 2-5 expand atoms 0 and 1 of every stage's four, warps 6-9 atoms 2 and 3; thread = weight
        // row of the tile.  (A second set of eight warps on alternate stages gained nothing: the sets share the SM's
        // integer pipes.)
        const int grp = (warp - 2) >> 2;
        const int quarter = warp & 3;           // the TMEM lanes this warp may access
        const int r = quarter * 32 + lane;      // weight row inside the tile
        const uint32_t m = 0x03030303u;
        int sit = 0;
        for (int t = blockIdx.x; t < total_tiles; t += gridDim.x) {
            for (int g = 0; g < stages; ++g, ++sit) {
                const int ps = sit % SM_PS, s = sit % SM_XS;
                mbar_wait(&p_full[ps], (sit / SM_PS) & 1, poisoned);
                const uint32_t row = smem_u32(p_ring + ps * SM_P_BYTES) + r * 128;
                // the row's 32 packed bytes of atom j: 16-byte chunks 2j, 2j + 1 (chunk c lies at c ^ (r & 7))
                uint4 pk[4];
#pragma unroll
                for (int c = 0; c < 4; ++c) pk[c] = lds128p(row + (((4 * grp + c) ^ (r & 7)) << 4));
                // the loads have returned once their values are used; the slot is handed back after the first atom
                if (sit >= SM_XS) mbar_wait(&st_free[s], ((sit / SM_XS) - 1) & 1, poisoned);
                tc_fence_after();
                const uint32_t dst = tmem_a + s * SM_A_COLS + grp * 64 + (static_cast<uint32_t>(quarter * 32) << 16);
#pragma unroll
                for (int jj = 0; jj < 2; ++jj) {
                    const uint32_t w[8] = {pk[2 * jj].x, pk[2 * jj].y, pk[2 * jj].z, pk[2 * jj].w,
                                           pk[2 * jj + 1].x, pk[2 * jj + 1].y, pk[2 * jj + 1].z, pk[2 * jj + 1].w};
                    uint32_t v[32];  // column c of the atom = its weights 4c .. 4c + 3
                    if (p.layout == WF_LAYOUT_WF16) {
#pragma unroll
                        for (int i = 0; i < 8; ++i) {
                            v[4 * i] = w[i] & m;
                            v[4 * i + 1] = (w[i] >> 2) & m;
                            v[4 * i + 2] = (w[i] >> 4) & m;
                            v[4 * i + 3] = (w[i] >> 6) & m;
                        }
                    } else {  // I2_S: byte b of the 32 holds weights b, b + 32, b + 64, b + 96 at bits 7:6, 5:4, 3:2, 1:0
#pragma unroll
                        for (int q = 0; q < 4; ++q)
#pragma unroll
                            for (int i = 0; i < 8; ++i) v[8 * q + i] = (w[i] >> (6 - 2 * q)) & m;
                    }
                    tmem_st32_nowait(dst + jj * 32, v);
                    if (jj == 1) {  // every packed byte of this warp's share is in registers or on its way to tensor memory
                        __syncwarp();
                        if (lane == 0) mbar_arrive(&p_empty[ps]);
                    }
                }
                asm volatile("tcgen05.wait::st.sync.aligned;\n" ::: "memory");
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(&a_full[s]);
            }
        }
    } else if (warp < 14 || (warp >= 15 && warp <= 18 && EPI_GROUPS == 2)) {
        // ---- epilogue: thread = weight row (TMEM lane), registers = tokens
        const int quarter = warp & 3;
        const int r = quarter * 32 + lane;
        const int egrp = warp >= 15 ? 1 : 0;
        const int et = egrp * 128 + (warp - (egrp ? 15 : 10)) * 32 + lane;  // 0 .. 128 * EPI_GROUPS - 1
        const int col0 = egrp * EPI_COLS;  // this group's first token column
        if (!p.x_ready) asm volatile("griddepcontrol.wait;\n" ::: "memory");
        int nt = 0, cur_zb = -1;
        for (int t = blockIdx.x; t < total_tiles; t += gridDim.x, ++nt) {
            const int z = t / tiles_per_problem, zb = t / p.tiles_n, tb = (t % tiles_per_problem) / p.tiles_n, rb = t % p.tiles_n;
            const int a = nt & 1;
            const int nrow = rb * SM_BM + r;
            const bool row_ok = nrow < p.N;
            const int tok_base = tb * NTOK;                 // first token of the block inside its problem
            const int mtok = min(NTOK, p.M - tok_base);     // valid tokens of the block
            if (zb != cur_zb) {  // uniform over the four warps: the constants of this token block
                asm volatile("bar.sync 2, %0;\n" ::"n"(128 * EPI_GROUPS) : "memory");  // nobody still reads the previous block's
                if (et < mtok) {
                    const int64_t tok = static_cast<int64_t>(z) * p.M + tok_base + et;
                    s_rowsum[et] = p.rowsum[tok];
                    s_inv[et] = p.x_scale ? __frcp_rn(p.x_scale[tok]) : 1.0f;
                }
                asm volatile("bar.sync 2, %0;\n" ::"n"(128 * EPI_GROUPS) : "memory");
                cur_zb = zb;
            }
            const float s_w = p.w_scale ? __ldg(p.w_scale + static_cast<int64_t>(z) * p.w_scale_stride) : p.w_scale_host;
            const bool has_bias = p.bias != nullptr;
            const float bias = (has_bias && row_ok) ? load1_rt(p.bias, p.bias_dtype, nrow) : 0.f;
            // These warps share their schedulers with the expansion warps: the per-token work is kept to a handful of
            // instructions (pointer increments, the output type decided outside the loop).
            const int64_t tok0 = static_cast<int64_t>(z) * p.M + tok_base;
            const bool fast16 = (p.y_dtype == WF_BF16 || p.y_dtype == WF_F16) && p.acc_out == nullptr;
            uint16_t* y16 = static_cast<uint16_t*>(p.y) + tok0 * p.ldy + nrow;
            const bool is_bf16 = p.y_dtype == WF_BF16;
            mbar_wait(&acc_full[a], (nt >> 1) & 1, poisoned);
            tc_fence_after();
#pragma unroll
            for (int c0 = col0; c0 < col0 + EPI_COLS; c0 += 16) {
                uint32_t v[16];
                if constexpr (NI == 1) {
                    tmem_ldn<16>(tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + a * ACC_BUF + c0, v);
                } else {  // the sum of the issuers' partial accumulators (an issuer without a stage in this tile wrote none)
#pragma unroll
                    for (int jt = 0; jt < 16; ++jt) v[jt] = 0;
                    const int r0 = static_cast<int>((static_cast<long long>(nt) * stages) % NI);
#pragma unroll
                    for (int i = 0; i < NI; ++i) {
                        const int g0 = i >= r0 ? i - r0 : i - r0 + NI;
                        if (g0 < stages) {
                            uint32_t u[16];
                            tmem_ldn<16>(tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + a * ACC_BUF + i * NTOK + c0, u);
#pragma unroll
                            for (int jt = 0; jt < 16; ++jt) v[jt] += u[jt];
                        }
                    }
                }
                if (c0 + 16 == col0 + EPI_COLS) {  // this group's columns are in registers: hand them back to the MMA warp
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&acc_empty[a]);
                }
                if (!row_ok) continue;
                if (fast16) {
                    epilogue16(v, s_rowsum + c0, s_inv + c0, s_w, has_bias, bias, is_bf16, y16 + static_cast<int64_t>(c0) * p.ldy, p.ldy, mtok - c0);
                } else {
#pragma unroll
                    for (int jt = 0; jt < 16; ++jt) {
                        const int tok_in = c0 + jt;
                        if (tok_in < mtok) {
                            const int64_t tok = tok0 + tok_in;
                            const int acc = static_cast<int>(v[jt]) - s_rowsum[tok_in];
                            float o = rescale(acc, s_inv[tok_in], s_w);
                            if (has_bias) o = __fadd_rn(o, bias);
                            store1_rt(p.y, p.y_dtype, tok * p.ldy + nrow, o);
                            if (p.acc_out) p.acc_out[tok * p.N + nrow] = acc;
                        }
                    }
                }
            }
        }
        // a grid that waited for nothing still ends after its predecessor: whoever waits for this grid may rely on
        // everything ahead of it in the stream
        if (p.x_ready) asm volatile("griddepcontrol.wait;\n" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    if (*poisoned) {
        // A CTA that gave up: nothing new was requested since, but copies and MMAs issued before may still be on their
        // way into this CTA's shared and tensor memory.  They take microseconds; the CTA keeps both for half a millisecond.
        for (int i = 0; i < 256; ++i) __nanosleep(2000);
        __syncthreads();
    }
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_base), "r"(512));
    }
}

// ---------------------------------------------------------------------------------------------------------
// Pair form, for many tokens.  The single-CTA kernel above is bound by L2 -> SM traffic: a 128 x 128 tile pulls 80 KB
// (64 KB of int8 tokens, 16 KB of packed weights) per 8.4 M multiply-adds.  Here the two CTAs of a cluster (two SMs)
// compute ONE tile of 256 weight rows x PR_N tokens with tcgen05.mma.cta_group::2: each CTA expands its own 128 weight
// rows into its own tensor memory (the A operand) and loads only ITS HALF of the token tile (PR_N / 2 tokens, the B
// operand of the pair is the union of the two halves), so the token bytes per multiply-add halve: 32 KB per 6.3 M.
// No load is multicast: every CTA fetches what it needs with an ordinary TMA copy; the copies of the token halves
// use the cta_group::2 form only so that both CTAs' bytes are counted on the barrier of the CTA that issues the MMAs.
//
// Per CTA: warp 0 TMA of its packed rows (stages of 512 K, each feeding two tensor-memory stages of 256 K); warp 14
// TMA of its token half; warps 2-5 / 6-9 expansion (first / second half of every packed stage); warp 1 of the LEADER
// (cluster rank 0) issues the MMAs of the pair and commits with a cluster multicast so that both CTAs see their
// buffers released; warps 10-13 and 15-18 epilogue of the CTA's own 128 rows x PR_N tokens.  Barriers that gather
// arrivals of both CTAs (token tile full, expanded weights ready, accumulator drained) live in the leader.
// Tensor memory: two accumulators of PR_N columns + a ring of PR_AS stages of expanded weights (256 K each) = 512 columns.
constexpr int PR_N = 192;                 // tokens per tile (the N of the MMA); a multiple of 32
constexpr int PR_HALF = PR_N / 2;         // tokens each CTA loads
constexpr int PR_PS = 4;                  // packed-weight stages (128 rows x 128 B = 16 KB, 512 K each)
constexpr int PR_XS = 3;                  // token stages (4 atoms of PR_HALF x 128 B = 48 KB, 512 K each: two tensor-memory stages)
constexpr int PR_AA = 2;                  // 128-byte atoms of K per tensor-memory stage (128 K each)
constexpr int PR_PARTS = 4 / PR_AA;       // tensor-memory stages that one packed stage (512 K) feeds
constexpr int PR_A_COLS = 32 * PR_AA;
constexpr int PR_ACC_COLS = 2 * PR_N;
constexpr int PR_AS = (512 - PR_ACC_COLS) / PR_A_COLS;  // ring of tensor-memory stages of expanded weights: what the accumulators leave
constexpr int PR_X_ATOM = PR_HALF * SM_BK;
constexpr int PR_X_BYTES = 4 * PR_X_ATOM;
constexpr size_t PR_SMEM = 1024 + PR_PS * SM_P_BYTES + PR_XS * PR_X_BYTES + 4096;
static_assert(PR_SMEM <= 227 * 1024, "shared memory of the pair form");
static_assert(PR_ACC_COLS + PR_AS * PR_A_COLS <= 512 && PR_N % 32 == 0 && PR_X_ATOM % 1024 == 0 && PR_AS % PR_PARTS == 0 && PR_PARTS == 2,
              "tensor memory / tile shape of the pair form");

__device__ __forceinline__ uint32_t cluster_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;\n" : "=r"(r));
    return r;
}
// the address of `p` (a shared-memory location of this CTA) in the CTA of rank `rank` of the cluster
__device__ __forceinline__ uint32_t map_to_rank(const void* p, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;\n" : "=r"(r) : "r"(smem_u32(p)), "r"(rank));
    return r;
}
// Arrival on a barrier of another CTA of the cluster.  What the barriers of this kernel order is tensor-memory traffic
// (tcgen05.st / tcgen05.ld completed by their own wait instructions and fenced with tcgen05.fence), not generic memory,
// so the arrival carries no cluster-scope release: that form cost about 1.5 k cycles per arrival in the expansion warps.
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
    asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];\n" ::"r"(cluster_addr) : "memory");
}
// commit of the pair's MMAs: one arrival on the barrier at this shared-memory offset in BOTH CTAs
__device__ __forceinline__ void tc_commit_pair(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;\n" ::"r"(smem_u32(bar)),
                 "h"(static_cast<uint16_t>(3))
                 : "memory");
}
// TMA copy into THIS CTA's shared memory whose bytes are counted on a barrier given as a cluster address (the leader's)
__device__ __forceinline__ void tma_load_2d_pair(void* dst, const void* tmap, int c0, int c1, uint32_t bar_cluster_addr) {
    asm volatile("cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];\n" ::"r"(
                     smem_u32(dst)),
                 "l"(reinterpret_cast<uint64_t>(tmap)), "r"(c0), "r"(c1), "r"(bar_cluster_addr)
                 : "memory");
}
__device__ __forceinline__ void mma_i8_ts_x4_pair(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc, uint32_t accumulate_first) {
    asm volatile(
        "{\n .reg .pred p, q;\n .reg .b32 a1, a2, a3;\n .reg .b64 b1, b2, b3;\n"
        " setp.ne.b32 p, %4, 0;\n setp.eq.b32 q, %5, %5;\n"
        " add.u32 a1, %1, 8;\n add.u32 a2, %1, 16;\n add.u32 a3, %1, 24;\n"
        " add.u64 b1, %2, 2;\n add.u64 b2, %2, 4;\n add.u64 b3, %2, 6;\n"
        " tcgen05.mma.cta_group::2.kind::i8 [%0], [%1], %2, %3, {%5, %5, %5, %5, %5, %5, %5, %5}, p;\n"
        " tcgen05.mma.cta_group::2.kind::i8 [%0], [a1], b1, %3, {%5, %5, %5, %5, %5, %5, %5, %5}, q;\n"
        " tcgen05.mma.cta_group::2.kind::i8 [%0], [a2], b2, %3, {%5, %5, %5, %5, %5, %5, %5, %5}, q;\n"
        " tcgen05.mma.cta_group::2.kind::i8 [%0], [a3], b3, %3, {%5, %5, %5, %5, %5, %5, %5, %5}, q;\n}\n" ::"r"(d_tmem),
        "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate_first), "r"(0u)
        : "memory");
}

__global__ void __launch_bounds__(SM_THREADS, 1)
    prefill_pair_kernel(const __grid_constant__ CUtensorMap tmap_x, const __grid_constant__ CUtensorMap tmap_p, const PrefillParams p) {
    constexpr int EPI_COLS = PR_N / 2;  // two epilogue warp groups, each takes half of the token columns
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
    uint8_t* p_ring = smem;                           // [PR_PS][128 rows x 128 B], 128-byte swizzle
    uint8_t* x_ring = p_ring + PR_PS * SM_P_BYTES;    // [PR_XS][2 atoms][PR_HALF rows x 128 B], 128-byte swizzle
    uint64_t* p_full = reinterpret_cast<uint64_t*>(x_ring + PR_XS * PR_X_BYTES);
    uint64_t* p_empty = p_full + PR_PS;
    uint64_t* x_full = p_empty + PR_PS;       // leader's copy: bytes of both CTAs' halves
    uint64_t* x_free = x_full + PR_XS;        // multicast commit: the token stage may be overwritten
    uint64_t* a_full = x_free + PR_XS;        // leader's copy: the expansion warps of both CTAs
    uint64_t* a_free = a_full + PR_AS;        // multicast commit: the tensor-memory stage may be overwritten
    uint64_t* acc_full = a_free + PR_AS;      // multicast commit: the accumulator of a tile is complete
    uint64_t* acc_empty = acc_full + 2;       // leader's copy: the epilogue warps of both CTAs
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
    volatile int* poisoned = reinterpret_cast<volatile int*>(tmem_slot + 1);
    // [PR_N] per-token constants of the epilogue's current token block, read as 16-byte vectors
    int* s_rowsum = reinterpret_cast<int*>((reinterpret_cast<uintptr_t>(tmem_slot + 2) + 15) & ~static_cast<uintptr_t>(15));
    float* s_inv = reinterpret_cast<float*>(s_rowsum + 256);  // [PR_N]

    // its dependents go when this grid's own wait is over (see the single form)
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const uint32_t rank = cluster_rank();     // 0: leader (issues the MMAs), 1: peer
    const int cluster_id = blockIdx.x >> 1, n_clusters = gridDim.x >> 1;
    // K is walked in packed stages of 512 and tensor-memory stages of 256; a stage that reaches past K is zero-filled by
    // the TMA unit on both operands.  Every tile runs an even number of tensor-memory stages, so a stage's half of its
    // packed stage and its expansion group are fixed by the parity of the running stage counter.
    const int pstages = (p.K + 511) / 512, astages = PR_PARTS * pstages;
    const int tiles_per_problem = p.tiles_m * p.tiles_n;  // token blocks of PR_N x row blocks of 256; row blocks vary fastest
    const int total_tiles = tiles_per_problem * p.batch;

    if (tid == 0) {
        for (int s = 0; s < PR_PS; ++s) {
            mbar_init(&p_full[s], 1);
            mbar_init(&p_empty[s], 8);
        }
        for (int s = 0; s < PR_XS; ++s) {
            mbar_init(&x_full[s], 1);
            mbar_init(&x_free[s], 1);
        }
        for (int s = 0; s < PR_AS; ++s) {
            mbar_init(&a_full[s], 8);
            mbar_init(&a_free[s], 1);
        }
        for (int a = 0; a < 2; ++a) {
            mbar_init(&acc_full[a], 1);
            mbar_init(&acc_empty[a], 16);
        }
        *poisoned = 0;
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
    if (warp == 1) {  // the same warp of both CTAs allocates the pair's tensor memory
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(smem_u32(tmem_slot)), "r"(512));
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;\n" ::);
    }
    tc_fence_before();
    __syncthreads();
    // both CTAs have initialised their barriers before either signals the other
    asm volatile("barrier.cluster.arrive.release.aligned;\n barrier.cluster.wait.acquire.aligned;\n" ::: "memory");
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    const uint32_t tmem_a = tmem_base + PR_ACC_COLS;  // PR_AS stages of PR_A_COLS columns

    if (warp == 0) {
        if (lane == 0) {  // this CTA's packed rows
            int psit = 0;
            for (int t = cluster_id; t < total_tiles; t += n_clusters) {
                const int z = t / tiles_per_problem, rb = t % p.tiles_n;
                const int row_w = z * p.N + rb * 256 + static_cast<int>(rank) * SM_BM;
                for (int g = 0; g < pstages; ++g, ++psit) {
                    const int s = psit % PR_PS;
                    if (psit >= PR_PS) mbar_wait(&p_empty[s], ((psit / PR_PS) - 1) & 1, poisoned);
                    mbar_expect_tx(&p_full[s], SM_P_BYTES);
                    tma_load_2d(p_ring + s * SM_P_BYTES, &tmap_p, g * 128, row_w, &p_full[s]);
                }
            }
        }
    } else if (warp == 14) {
        if (lane == 0) {  // this CTA's half of the token tile; the bytes are counted on the leader's barrier
            asm volatile("griddepcontrol.wait;\n" ::: "memory");
            asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory");
            int xsit = 0;
            for (int t = cluster_id; t < total_tiles; t += n_clusters) {
                const int row_x = (t / tiles_per_problem) * p.M + ((t % tiles_per_problem) / p.tiles_n) * PR_N + static_cast<int>(rank) * PR_HALF;
                for (int g = 0; g < pstages; ++g, ++xsit) {
                    const int s = xsit % PR_XS;
                    if (xsit >= PR_XS) mbar_wait(&x_free[s], ((xsit / PR_XS) - 1) & 1, poisoned);
                    if (rank == 0) mbar_expect_tx(&x_full[s], 2 * PR_X_BYTES);
                    const uint32_t bar = map_to_rank(&x_full[s], 0);
#pragma unroll
                    for (int j = 0; j < 4; ++j)  // an atom that lies past K arrives as zeros
                        tma_load_2d_pair(x_ring + s * PR_X_BYTES + j * PR_X_ATOM, &tmap_x, (g * 4 + j) * SM_BK, row_x, bar);
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0 && rank == 0) {
            // D = s32, A = unsigned 8-bit (codes, from tensor memory), B = signed 8-bit (tokens, K-major), N = PR_N, M = 256 over the pair
            const uint32_t idesc = (2u << 4) | (0u << 7) | (1u << 10) | (static_cast<uint32_t>(PR_N >> 3) << 17) | (static_cast<uint32_t>(256 >> 4) << 24);
            uint64_t bdesc[PR_XS][4];  // per token stage and 128-byte atom of K
#pragma unroll
            for (int s = 0; s < PR_XS; ++s)
#pragma unroll
                for (int j = 0; j < 4; ++j) bdesc[s][j] = smem_desc_sw128(smem_u32(x_ring + s * PR_X_BYTES + j * PR_X_ATOM));
            int sit = 0, nt = 0;
            for (int t = cluster_id; t < total_tiles; t += n_clusters, ++nt) {
                const int a = nt & 1;
                if (nt >= 2) mbar_wait(&acc_empty[a], ((nt >> 1) - 1) & 1, poisoned);
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + a * PR_N;
                for (int g = 0; g < astages; ++g, ++sit) {
                    // token stage = packed stage = PR_PARTS tensor-memory stages; `part` = which of them
                    const int xsit = sit / PR_PARTS, xs = xsit % PR_XS, part = sit % PR_PARTS, as = sit % PR_AS;
                    if (part == 0) mbar_wait(&x_full[xs], (xsit / PR_XS) & 1, poisoned);
                    mbar_wait(&a_full[as], (sit / PR_AS) & 1, poisoned);
                    tc_fence_after();
                    const uint32_t a_stage = tmem_a + as * PR_A_COLS;
#pragma unroll
                    for (int ss = 0; ss < PR_XS; ++ss) {
                        if (ss == xs) {
#pragma unroll
                            for (int pp = 0; pp < PR_PARTS; ++pp) {
                                if (pp == part) {
#pragma unroll
                                    for (int j = 0; j < PR_AA; ++j)
                                        mma_i8_ts_x4_pair(d_tmem, a_stage + j * 32, bdesc[ss][pp * PR_AA + j], idesc, (g | j) ? 1u : 0u);
                                }
                            }
                        }
                    }
                    tc_commit_pair(&a_free[as]);
                    if (part == PR_PARTS - 1) tc_commit_pair(&x_free[xs]);  // the whole token stage has been consumed
                }
                tc_commit_pair(&acc_full[a]);
            }
        }
    } else if (warp < 10) {
        // ---- expansion: the two groups alternate tensor-memory stages; thread = weight row
        const int grp = (warp - 2) >> 2;
        const int quarter = warp & 3;
        const int r = quarter * 32 + lane;
        const uint32_t m = 0x03030303u;
        int sit = grp;  // this group's tensor-memory stages: grp, grp + 2, ...
        for (int t = cluster_id; t < total_tiles; t += n_clusters) {
            for (int g = grp; g < astages; g += 2, sit += 2) {
                const int psit = sit / PR_PARTS, ps = psit % PR_PS, part = sit % PR_PARTS, as = sit % PR_AS;
                mbar_wait(&p_full[ps], (psit / PR_PS) & 1, poisoned);
                // The packed bytes are expanded into registers BEFORE the tensor-memory stage is known to be free: what
                // remains between "the MMAs of the previous use have completed" and "the next MMAs may start" is the
                // tcgen05.st and its wait.
                const uint32_t row = smem_u32(p_ring + ps * SM_P_BYTES) + r * 128;
                uint32_t v[PR_AA][32];
#pragma unroll
                for (int jj = 0; jj < PR_AA; ++jj) {
                    const int j = part * PR_AA + jj;  // atom of the packed stage
                    const uint4 lo = lds128p(row + (((2 * j) ^ (r & 7)) << 4));
                    const uint4 hi = lds128p(row + (((2 * j + 1) ^ (r & 7)) << 4));
                    const uint32_t w[8] = {lo.x, lo.y, lo.z, lo.w, hi.x, hi.y, hi.z, hi.w};
                    if (p.layout == WF_LAYOUT_WF16) {
#pragma unroll
                        for (int i = 0; i < 8; ++i) {
                            v[jj][4 * i] = w[i] & m;
                            v[jj][4 * i + 1] = (w[i] >> 2) & m;
                            v[jj][4 * i + 2] = (w[i] >> 4) & m;
                            v[jj][4 * i + 3] = (w[i] >> 6) & m;
                        }
                    } else {
#pragma unroll
                        for (int q = 0; q < 4; ++q)
#pragma unroll
                            for (int i = 0; i < 8; ++i) v[jj][8 * q + i] = (w[i] >> (6 - 2 * q)) & m;
                    }
                }
                __syncwarp();
                // this group's last part of the packed stage: its rows are in registers
                if (lane == 0 && part + 2 >= PR_PARTS) mbar_arrive(&p_empty[ps]);
                if (sit >= PR_AS) mbar_wait(&a_free[as], ((sit / PR_AS) - 1) & 1, poisoned);
                tc_fence_after();
                const uint32_t dst = tmem_a + as * PR_A_COLS + (static_cast<uint32_t>(quarter * 32) << 16);
#pragma unroll
                for (int jj = 0; jj < PR_AA; ++jj) tmem_st32_nowait(dst + jj * 32, v[jj]);
                asm volatile("tcgen05.wait::st.sync.aligned;\n" ::: "memory");
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive_cluster(map_to_rank(&a_full[as], 0));  // expanded rows of this CTA are in its tensor memory
            }
        }
    } else if (warp < 14 || warp >= 15) {
        // ---- epilogue of this CTA's 128 rows: thread = weight row (TMEM lane), registers = tokens
        const int quarter = warp & 3;
        const int r = quarter * 32 + lane;
        const int egrp = warp >= 15 ? 1 : 0;
        const int et = egrp * 128 + (warp - (egrp ? 15 : 10)) * 32 + lane;  // 0 .. 255
        const int col0 = egrp * EPI_COLS;
        const uint32_t acc_empty_leader0 = map_to_rank(&acc_empty[0], 0), acc_empty_leader1 = map_to_rank(&acc_empty[1], 0);
        asm volatile("griddepcontrol.wait;\n" ::: "memory");
        int nt = 0, cur_zb = -1;
        for (int t = cluster_id; t < total_tiles; t += n_clusters, ++nt) {
            const int z = t / tiles_per_problem, zb = t / p.tiles_n, tb = (t % tiles_per_problem) / p.tiles_n, rb = t % p.tiles_n;
            const int a = nt & 1;
            const int nrow = rb * 256 + static_cast<int>(rank) * SM_BM + r;
            const bool row_ok = nrow < p.N;
            const int tok_base = tb * PR_N;
            const int mtok = min(PR_N, p.M - tok_base);
            if (zb != cur_zb) {
                asm volatile("bar.sync 2, 256;\n" ::: "memory");
                if (et < mtok) {
                    const int64_t tok = static_cast<int64_t>(z) * p.M + tok_base + et;
                    s_rowsum[et] = p.rowsum[tok];
                    s_inv[et] = p.x_scale ? __frcp_rn(p.x_scale[tok]) : 1.0f;
                }
                asm volatile("bar.sync 2, 256;\n" ::: "memory");
                cur_zb = zb;
            }
            const float s_w = p.w_scale ? __ldg(p.w_scale + static_cast<int64_t>(z) * p.w_scale_stride) : p.w_scale_host;
            const bool has_bias = p.bias != nullptr;
            const float bias = (has_bias && row_ok) ? load1_rt(p.bias, p.bias_dtype, nrow) : 0.f;
            const int64_t tok0 = static_cast<int64_t>(z) * p.M + tok_base;
            const bool fast16 = (p.y_dtype == WF_BF16 || p.y_dtype == WF_F16) && p.acc_out == nullptr;
            uint16_t* y16 = static_cast<uint16_t*>(p.y) + tok0 * p.ldy + nrow;
            const bool is_bf16 = p.y_dtype == WF_BF16;
            mbar_wait(&acc_full[a], (nt >> 1) & 1, poisoned);
            tc_fence_after();
#pragma unroll
            for (int c0 = col0; c0 < col0 + EPI_COLS; c0 += 16) {
                uint32_t v[16];
                tmem_ldn<16>(tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + a * PR_N + c0, v);
                if (c0 + 16 == col0 + EPI_COLS) {  // this group's columns are in registers: hand them back to the MMA thread
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive_cluster(a ? acc_empty_leader1 : acc_empty_leader0);
                }
                if (!row_ok) continue;
                if (fast16) {
                    epilogue16(v, s_rowsum + c0, s_inv + c0, s_w, has_bias, bias, is_bf16, y16 + static_cast<int64_t>(c0) * p.ldy, p.ldy, mtok - c0);
                } else {
#pragma unroll
                    for (int jt = 0; jt < 16; ++jt) {
                        const int tok_in = c0 + jt;
                        if (tok_in < mtok) {
                            const int64_t tok = tok0 + tok_in;
                            const int acc = static_cast<int>(v[jt]) - s_rowsum[tok_in];
                            float o = rescale(acc, s_inv[tok_in], s_w);
                            if (has_bias) o = __fadd_rn(o, bias);
                            store1_rt(p.y, p.y_dtype, tok * p.ldy + nrow, o);
                            if (p.acc_out) p.acc_out[tok * p.N + nrow] = acc;
                        }
                    }
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    // neither CTA leaves (nor frees the pair's tensor memory) while the other may still signal it
    asm volatile("barrier.cluster.arrive.release.aligned;\n barrier.cluster.wait.acquire.aligned;\n" ::: "memory");
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_base), "r"(512));
    }
}

// row sums of an int8 matrix (for activations that arrive already quantized)
__global__ void rowsum_i8_kernel(const int8_t* __restrict__ q, int64_t ldq, int K, int32_t* __restrict__ rowsum) {
    const int64_t m = blockIdx.x;
    int s = 0;
    for (int k = threadIdx.x * 16; k < K; k += blockDim.x * 16) {
        const uint4 v = __ldg(reinterpret_cast<const uint4*>(q + m * ldq + k));
        s += __dp4a(static_cast<int>(v.x), 0x01010101, 0) + __dp4a(static_cast<int>(v.y), 0x01010101, 0) +
             __dp4a(static_cast<int>(v.z), 0x01010101, 0) + __dp4a(static_cast<int>(v.w), 0x01010101, 0);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    __shared__ int sh[8];
    if ((threadIdx.x & 31) == 0) sh[threadIdx.x >> 5] = s;
    __syncthreads();
    if (threadIdx.x == 0) {
        int t = 0;
        for (int i = 0; i < (blockDim.x >> 5); ++i) t += sh[i];
        rowsum[m] = t;
    }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn pf_encode_fn() {
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        void* ptr = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(ptr);
    }
    return fn;
}

static size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

}  // namespace wf

using namespace wf;

extern "C" int wf_prefill_status_fetch(int* out) {
    WF_CUDA(cudaMemcpyFromSymbol(out, g_prefill_status, sizeof(int)));
    if (*out) {
        int zero = 0;
        WF_CUDA(cudaMemcpyToSymbol(g_prefill_status, &zero, sizeof(int)));
    }
    return WF_OK;
}

// workspace: int8 activations [M, K] | multipliers [M] | row sums [M]
extern "C" size_t wf_prefill_workspace_bytes(int64_t M, int64_t K) {
    if (M <= 0 || K <= 0) return 0;
    return align_up(static_cast<size_t>(M) * K, 256) + 2 * align_up(static_cast<size_t>(M) * 4, 256);
}

// `batch` independent problems stacked along the rows: tokens [batch*M, K], weights [batch*N, K/4],
// outputs [batch*M, N]; problem z uses the weight scale w_scale[z * w_scale_stride].
static int prefill_impl(const char* who, const void* x, int x_dtype, int64_t ldx, const float* x_scale, const uint8_t* codes,
                        int layout, const float* w_scale, int64_t w_scale_stride, float w_scale_host, const void* bias,
                        int bias_dtype, void* y, int y_dtype, int64_t ldy, int32_t* acc_out, int64_t batch, int64_t M_one,
                        int64_t N, int64_t K, float eps, void* workspace, size_t workspace_bytes, unsigned flags, void* stream) {
    const int64_t M = batch * M_one;  // rows of the stacked activations
    if (int rc = wf_check_linear_args(who, x, x_dtype, ldx, x_scale, codes, layout, bias, bias_dtype, y, y_dtype, ldy, M, N, K))
        return rc;
    WF_REQUIRE(batch >= 1 && batch * N < (1LL << 31), "%s: batch out of range", who);
    WF_REQUIRE(workspace && reinterpret_cast<uintptr_t>(workspace) % 256 == 0, "wf_bitlinear_prefill: workspace must be 256-byte aligned");
    if (workspace_bytes < wf_prefill_workspace_bytes(M, K))
        return fail(WF_E_SCRATCH, "wf_bitlinear_prefill: workspace of %zu bytes, need %zu", workspace_bytes,
                    wf_prefill_workspace_bytes(M, K));
    if (int rc = require_device()) return rc;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    uint8_t* ws = static_cast<uint8_t*>(workspace);
    int8_t* wq = reinterpret_cast<int8_t*>(ws);
    float* wscale = reinterpret_cast<float*>(ws + align_up(static_cast<size_t>(M) * K, 256));
    int32_t* wsum = reinterpret_cast<int32_t*>(ws + align_up(static_cast<size_t>(M) * K, 256) + align_up(static_cast<size_t>(M) * 4, 256));

    const int8_t* q = nullptr;
    const float* qs = nullptr;
    int64_t ldq = K;
    if (flags & WF_FLAG_WS_READY) {  // wf_prefill_quantize filled the workspace earlier in the stream
        q = wq;
        qs = wscale;
    } else if (x_dtype != WF_I8) {
        if (int rc = wf_act_quant_i8(x, x_dtype, M, K, ldx, WF_ACT_PER_TOKEN, eps, wq, wscale, wsum, stream)) return rc;
        q = wq;
        qs = wscale;
    } else {
        q = static_cast<const int8_t*>(x);
        qs = x_scale;
        ldq = ldx;
        rowsum_i8_kernel<<<static_cast<unsigned>(M), 128, 0, st>>>(q, ldq, static_cast<int>(K), wsum);
        WF_CUDA(cudaGetLastError());
    }

    EncodeTiledFn enc = pf_encode_fn();
    if (!enc) return fail(WF_E_DEVICE, "cuTensorMapEncodeTiled is not available in this driver");
    const int ntok = M_one <= 16 ? 16 : (M_one <= 32 ? 32 : (M_one <= 64 ? 64 : 128));
    const int sms = num_sms();
    // Single form (one CTA per 128 x 128 tile) unless the caller asks for the pair form (two CTAs per 256 x PR_N tile):
    // measured on B200 at M = 512 ... 8192 on the three sweep shapes the single form is the faster one everywhere
    // (1.41 / 1.68 / 2.13 POPS against 1.22 / 1.58 / 1.79 at M = 8192; a pair tile of 128 tokens with a ring of four
    // tensor-memory stages was slower still), although the pair form pulls half the token bytes from L2.
    bool pair = false;
    if (ntok == 128 && (flags & WF_FLAG_PREFILL_PAIR) && !(flags & WF_FLAG_PREFILL_SINGLE)) pair = sms >= 2;
    alignas(64) CUtensorMap tmap_a, tmap_p;
    const cuuint32_t ones[2] = {1, 1};
    {
        const cuuint64_t dims[2] = {static_cast<cuuint64_t>(K), static_cast<cuuint64_t>(M)};
        const cuuint64_t strides[1] = {static_cast<cuuint64_t>(ldq)};
        const cuuint32_t box[2] = {SM_BK, static_cast<cuuint32_t>(pair ? PR_HALF : ntok)};
        CUresult r = enc(&tmap_a, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<int8_t*>(q), dims, strides, box, ones,
                         CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                         CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_SUCCESS) return fail(WF_E_DEVICE, "cuTensorMapEncodeTiled (activations) failed with %d", (int)r);
    }
    {
        const cuuint64_t dims[2] = {static_cast<cuuint64_t>(K / 4), static_cast<cuuint64_t>(batch * N)};
        const cuuint64_t strides[1] = {static_cast<cuuint64_t>(K / 4)};
        const cuuint32_t box[2] = {SM_PK * SM_BK / 4, SM_BM};
        CUresult r = enc(&tmap_p, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<uint8_t*>(codes), dims, strides, box, ones,
                         CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                         CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_SUCCESS) return fail(WF_E_DEVICE, "cuTensorMapEncodeTiled (packed weights) failed with %d", (int)r);
    }
    PrefillParams pp;
    pp.x_scale = qs; pp.rowsum = wsum; pp.w_scale = w_scale; pp.w_scale_host = w_scale_host; pp.bias = bias;
    pp.bias_dtype = bias_dtype; pp.y = y; pp.y_dtype = y_dtype; pp.ldy = ldy; pp.acc_out = acc_out;
    pp.M = static_cast<int>(M_one); pp.N = static_cast<int>(N); pp.K = static_cast<int>(K); pp.layout = layout;
    pp.batch = static_cast<int>(batch); pp.w_scale_stride = static_cast<int>(w_scale_stride);
    pp.tiles_m = static_cast<int>(pair ? (M_one + PR_N - 1) / PR_N : (M_one + ntok - 1) / ntok);
    pp.tiles_n = static_cast<int>(pair ? (N + 255) / 256 : (N + SM_BM - 1) / SM_BM);
    pp.x_ready = ((flags & WF_FLAG_WS_READY) && (flags & WF_FLAG_X_READY) && !pair) ? 1 : 0;
    static PerDeviceOnce configured;  // the attribute is a per-device setting
    const int dev_now = current_device();
    if (configured.needs(dev_now)) {
        WF_CUDA(cudaFuncSetAttribute(prefill_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(PR_SMEM)));
        WF_CUDA(cudaFuncSetAttribute(prefill_kernel<16>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(sm_smem<16>())));
        WF_CUDA(cudaFuncSetAttribute(prefill_kernel<32>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(sm_smem<32>())));
        WF_CUDA(cudaFuncSetAttribute(prefill_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(sm_smem<64>())));
        WF_CUDA(cudaFuncSetAttribute(prefill_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(sm_smem<128>())));
        configured.mark(dev_now);
    }
    const long long tiles = static_cast<long long>(pp.tiles_m) * pp.tiles_n * pp.batch;
    cudaLaunchConfig_t lc = {};
    lc.gridDim = dim3(static_cast<unsigned>(tiles < sms ? tiles : sms));
    lc.blockDim = dim3(SM_THREADS);
    lc.stream = st;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    lc.attrs = attr;
    lc.numAttrs = 1;
    if (pair) {
        const long long clusters = tiles < sms / 2 ? tiles : sms / 2;
        lc.gridDim = dim3(static_cast<unsigned>(2 * clusters));
        attr[1].id = cudaLaunchAttributeClusterDimension;
        attr[1].val.clusterDim.x = 2;
        attr[1].val.clusterDim.y = 1;
        attr[1].val.clusterDim.z = 1;
        lc.numAttrs = 2;
        lc.dynamicSmemBytes = PR_SMEM;
        WF_CUDA(cudaLaunchKernelEx(&lc, prefill_pair_kernel, tmap_a, tmap_p, pp));
    } else if (ntok == 16) {
        lc.blockDim = dim3(sm_threads<16>());
        lc.dynamicSmemBytes = sm_smem<16>();
        WF_CUDA(cudaLaunchKernelEx(&lc, prefill_kernel<16>, tmap_a, tmap_p, pp));
    } else if (ntok == 32) {
        lc.blockDim = dim3(sm_threads<32>());
        lc.dynamicSmemBytes = sm_smem<32>();
        WF_CUDA(cudaLaunchKernelEx(&lc, prefill_kernel<32>, tmap_a, tmap_p, pp));
    } else if (ntok == 64) {
        lc.blockDim = dim3(sm_threads<64>());
        lc.dynamicSmemBytes = sm_smem<64>();
        WF_CUDA(cudaLaunchKernelEx(&lc, prefill_kernel<64>, tmap_a, tmap_p, pp));
    } else {
        lc.dynamicSmemBytes = sm_smem<128>();
        WF_CUDA(cudaLaunchKernelEx(&lc, prefill_kernel<128>, tmap_a, tmap_p, pp));
    }
    return WF_OK;
}

extern "C" int wf_bitlinear_prefill(const void* x, int x_dtype, int64_t ldx, const float* x_scale, const uint8_t* codes,
                                    int layout, const float* w_scale, float w_scale_host, const void* bias, int bias_dtype,
                                    void* y, int y_dtype, int64_t ldy, int32_t* acc_out, int64_t M, int64_t N, int64_t K,
                                    float eps, void* workspace, size_t workspace_bytes, unsigned flags, void* stream) {
    return prefill_impl("wf_bitlinear_prefill", x, x_dtype, ldx, x_scale, codes, layout, w_scale, 0, w_scale_host, bias,
                        bias_dtype, y, y_dtype, ldy, acc_out, 1, M, N, K, eps, workspace, workspace_bytes, flags, stream);
}

extern "C" int wf_bitlinear_prefill_batched(const void* x, int x_dtype, int64_t ldx, const uint8_t* codes, int layout,
                                            const float* w_scale, int64_t w_scale_stride, void* y, int y_dtype, int64_t ldy,
                                            int32_t* acc_out, int64_t batch, int64_t M, int64_t N, int64_t K, float eps,
                                            void* workspace, size_t workspace_bytes, unsigned flags, void* stream) {
    WF_REQUIRE(w_scale, "wf_bitlinear_prefill_batched: w_scale must point to the per-problem scales");
    WF_REQUIRE(x_dtype != WF_I8, "wf_bitlinear_prefill_batched: takes floating-point activations");
    return prefill_impl("wf_bitlinear_prefill_batched", x, x_dtype, ldx, nullptr, codes, layout, w_scale, w_scale_stride, 0.f,
                        nullptr, 0, y, y_dtype, ldy, acc_out, batch, M, N, K, eps, workspace, workspace_bytes,
                        flags & (WF_FLAG_WS_READY | WF_FLAG_X_READY), stream);
}

int wf_act_quant_token_ready(const void* x, int x_dtype, int64_t M, int64_t K, int64_t ldx, float eps, int8_t* q, float* scale,
                             int32_t* rowsum, int x_ready, void* stream);

extern "C" int wf_prefill_quantize(const void* x, int x_dtype, int64_t ldx, int64_t M, int64_t K, float eps, void* workspace,
                                   size_t workspace_bytes, unsigned flags, void* stream) {
    WF_REQUIRE(x && x_dtype != WF_I8, "wf_prefill_quantize: takes floating-point activations");
    WF_REQUIRE(M > 0 && K > 0 && K % 4 == 0 && ldx >= K, "wf_prefill_quantize: bad shape");
    WF_REQUIRE(workspace && reinterpret_cast<uintptr_t>(workspace) % 256 == 0, "wf_prefill_quantize: workspace must be 256-byte aligned");
    if (workspace_bytes < wf_prefill_workspace_bytes(M, K))
        return wf::fail(WF_E_SCRATCH, "wf_prefill_quantize: workspace of %zu bytes, need %zu", workspace_bytes,
                        wf_prefill_workspace_bytes(M, K));
    uint8_t* ws = static_cast<uint8_t*>(workspace);
    const size_t qb = wf::align_up(static_cast<size_t>(M) * K, 256), sb = wf::align_up(static_cast<size_t>(M) * 4, 256);
    return wf_act_quant_token_ready(x, x_dtype, M, K, ldx, eps, reinterpret_cast<int8_t*>(ws), reinterpret_cast<float*>(ws + qb),
                                    reinterpret_cast<int32_t*>(ws + qb + sb), (flags & WF_FLAG_X_READY) ? 1 : 0, stream);
}
