// Decode-step attention over the bf16 KV cache: one new token per sequence, grouped-query heads, causal by
// construction (the cache holds only positions <= the current one).  HBM-bound: every key and value of the context
// is read once per step, so the kernel is a streaming reduction.
//
//   out[b, h, :] = softmax_t(scale * q[b, h, :] . K[b, kv(h), t, :]) @ V[b, kv(h), t, :]      t < n_valid
//
// Work split.  A unit is one (sequence, KV head); a CTA (4 warps) serves ALL query heads of the unit's group at once,
// so K and V are read once for the group.  The 64-position tiles of all units form one unit-major sequence that is cut
// into equal contiguous ranges, one per persistent CTA (two per SM): the load is balanced whatever the batch, and a
// CTA keeps streaming across unit boundaries.  Where a unit is shared by several CTAs (small batches: the context of
// one unit is spread over many CTAs) each leaves an un-normalised partial result with its running maximum and sum in a
// workspace, and the last of them to finish (an atomic ticket) merges - no second launch.
//
// Data path.  K and V tiles of 64 positions stream through a 3-stage ring in shared memory with 16-byte
// cp.async copies (rows of D bf16, 16-byte chunks XOR-swizzled by the row so that ldmatrix reads are conflict
// free).  Each warp takes 16 positions of a tile: S = Q K^T on mma.sync.m16n8k16 bf16 with the group's query heads
// as the (zero-padded) 16 rows, fp32 online softmax with exp2, P V on the same instruction with V read through
// ldmatrix.trans.  Two CTAs fit an SM (about 108 KB each), which keeps about 128 KB of loads in flight per SM.
#include "wf_common.cuh"

namespace wf {

constexpr int AT_WARPS = 4;
constexpr int AT_THREADS = AT_WARPS * 32;
constexpr int AT_TILE = 64;   // positions per stage
constexpr int AT_STAGES = 3;
constexpr int AT_MAX_SPLITS = 64;

__device__ __forceinline__ uint32_t at_smem(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, bool valid) {
    const int n = valid ? 16 : 0;  // zero-fill beyond the valid length
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(dst), "l"(src), "r"(n) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;\n" ::"n"(N) : "memory");
}
__device__ __forceinline__ void ldsm_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_trans(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void mma_bf16(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack2_bf16(float lo, float hi) {
    const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&v);
}

struct AttnParams {
    const __nv_bfloat16* q;    // [B, nq * D]
    const __nv_bfloat16* k;    // [B, nkv, T, D]
    const __nv_bfloat16* v;
    const int64_t* pos;        // device scalar: positions 0 .. *pos are valid (nullable: all T)
    __nv_bfloat16* out;        // [B, nq * D]
    float* part_o;             // [units, kmax, G, D]  un-normalised partial outputs
    float* part_ml;            // [units, kmax, G, 2]  running maximum (log2 domain) and sum
    int* tickets;              // [units]
    int nq, nkv, T, units, kmax;
    int unit_aligned;          // CTA ranges end on unit boundaries (many units): no unit is shared, no tickets
    float scale_log2;          // softmax scale * log2(e)
};

// byte offset of the 16-byte chunk `c` of row `r` in a tile whose rows hold D bf16
template <int D>
__device__ __forceinline__ uint32_t tile_off(int r, int c) {
    return static_cast<uint32_t>(r * (D * 2) + ((c ^ (r & 7)) << 4));
}

// Persistent form: the tiles of all (sequence, KV head) units form one sequence (unit-major) that is cut into equal
// contiguous ranges, one per CTA; a CTA streams its range through the ring without draining at a unit boundary
// (the copies of the next unit's first tiles are in flight while the finished unit is merged and stored).  A unit whose
// tiles fall into several ranges is merged by the last of those CTAs to finish.
template <int D>
__global__ void __launch_bounds__(AT_THREADS, 2) attn_decode_kernel(const AttnParams p) {
    constexpr int ROW_BYTES = D * 2, CHUNKS = D / 8;       // 16-byte chunks per row
    constexpr int TILE_BYTES = AT_TILE * ROW_BYTES;        // one of K or V
    constexpr int KSTEPS = D / 16, NTILES = D / 8, HALF_NT = NTILES / 2;
    extern __shared__ __align__(128) uint8_t smem[];
    uint8_t* q_s = smem;                                   // [16 rows][D] bf16, swizzled like the tiles
    uint8_t* ring = smem + 16 * ROW_BYTES;                 // [AT_STAGES][K tile | V tile]
    float* red_o = reinterpret_cast<float*>(ring + AT_STAGES * 2 * TILE_BYTES);  // [AT_WARPS][8 rows][D / 2]
    float* red_ml = red_o + AT_WARPS * 8 * (D / 2);                              // [AT_WARPS][8 rows][2]
    __shared__ int s_last;
    asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory");
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int G = p.nq / p.nkv;
    // q, the cache and the position are written by the previous kernels of the stream
    asm volatile("griddepcontrol.wait;\n" ::: "memory");
    int n_valid = p.T;
    if (p.pos) {
        const int64_t pv = *p.pos + 1;
        n_valid = pv < p.T ? static_cast<int>(pv) : p.T;
    }
    const int tpu = (n_valid + AT_TILE - 1) / AT_TILE;                    // tiles per unit
    const int total = p.units * tpu;                                      // < 2^31 (checked on the host)
    int R = (total + gridDim.x - 1) / gridDim.x;                          // tiles per CTA
    if (p.unit_aligned) R = (R + tpu - 1) / tpu * tpu;
    const int gt0 = blockIdx.x * R;
    const int gt1 = min(gt0 + R, total);
    if (gt0 >= gt1) return;

    int iu = gt0 / tpu, itile = gt0 - iu * tpu, islot = 0;  // cursor of the next tile to request: unit, tile, ring slot
    auto issue_tile = [&](int gt) {
        if (gt < gt1) {
            const int u = iu, tile = itile;
            uint8_t* ks = ring + islot * 2 * TILE_BYTES;
            if (++itile == tpu) { itile = 0; ++iu; }
            if (++islot == AT_STAGES) islot = 0;
            uint8_t* vs = ks + TILE_BYTES;
            const __nv_bfloat16* kbase = p.k + static_cast<int64_t>(u) * p.T * D;  // units are laid out [B, nkv] like the cache
            const __nv_bfloat16* vbase = p.v + static_cast<int64_t>(u) * p.T * D;
            const int t0 = tile * AT_TILE;
            for (int i = tid; i < AT_TILE * CHUNKS; i += AT_THREADS) {
                const int r = i / CHUNKS, c = i % CHUNKS;
                const bool ok = t0 + r < n_valid;
                const int64_t src = static_cast<int64_t>(ok ? t0 + r : 0) * D + c * 8;
                cp_async16(at_smem(ks) + tile_off<D>(r, c), kbase + src, ok);
                cp_async16(at_smem(vs) + tile_off<D>(r, c), vbase + src, ok);
            }
        }
        cp_async_commit();  // one group per tile slot, also when empty: the wait counts stay uniform
    };
    issue_tile(gt0);
    issue_tile(gt0 + 1);

    const int g = lane >> 2, t4 = lane & 3;
    uint32_t qa[KSTEPS][4];
    float o[NTILES][4];
    float m_run = -INFINITY, l_run = 0.f;  // of query row g (rows g + 8 are padding)

    int u = gt0 / tpu, tile = gt0 - u * tpu - 1, slot_c = AT_STAGES - 1;  // cursor of the tile being consumed
    for (int gt = gt0; gt < gt1; ++gt) {
        if (++tile == tpu) { tile = 0; ++u; }
        if (++slot_c == AT_STAGES) slot_c = 0;
        if (gt == gt0 || tile == 0) {
            // ---- a new unit: its query rows (rows >= G are zero) as A fragments, fresh running state
            for (int i = tid; i < 16 * CHUNKS; i += AT_THREADS) {
                const int r = i / CHUNKS, c = i % CHUNKS;
                uint4 val = make_uint4(0, 0, 0, 0);
                if (r < G) val = *reinterpret_cast<const uint4*>(p.q + (static_cast<int64_t>(u) * G + r) * D + c * 8);
                *reinterpret_cast<uint4*>(q_s + tile_off<D>(r, c)) = val;
            }
            __syncthreads();
            {   // matrices (rows 0-7, k 0-7), (rows 8-15, k 0-7), (rows 0-7, k 8-15), (rows 8-15, k 8-15)
                const int r = (lane & 7) + ((lane >> 3) & 1) * 8, half = lane >> 4;
#pragma unroll
                for (int s = 0; s < KSTEPS; ++s) ldsm_x4(at_smem(q_s) + tile_off<D>(r, 2 * s + half), qa[s][0], qa[s][1], qa[s][2], qa[s][3]);
            }
#pragma unroll
            for (int j = 0; j < NTILES; ++j) o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.f;
            m_run = -INFINITY;
            l_run = 0.f;
        }
        issue_tile(gt + 2);
        cp_async_wait<2>();  // the copies of this tile have landed (two younger groups may be in flight)
        __syncthreads();
        const uint8_t* ks = ring + slot_c * 2 * TILE_BYTES;
        const uint8_t* vs = ks + TILE_BYTES;
        const int row0 = warp * 16;                  // this warp's 16 positions of the tile
        const int tpos = tile * AT_TILE + row0;      // position of its first one
        if (tpos < n_valid) {
            // ---- S = Q K^T: two n-tiles of 8 positions
            float s0[4] = {0.f, 0.f, 0.f, 0.f}, s1[4] = {0.f, 0.f, 0.f, 0.f};
            {
                // matrices: (positions 0-7, k 0-7), (positions 0-7, k 8-15), (positions 8-15, k 0-7), (positions 8-15, k 8-15)
                const int r = row0 + (lane & 7) + (lane >> 4) * 8, half = (lane >> 3) & 1;
#pragma unroll
                for (int s = 0; s < KSTEPS; ++s) {
                    uint32_t b0, b1, b2, b3;
                    ldsm_x4(at_smem(ks) + tile_off<D>(r, 2 * s + half), b0, b1, b2, b3);
                    mma_bf16(s0, qa[s][0], qa[s][1], qa[s][2], qa[s][3], b0, b1);
                    mma_bf16(s1, qa[s][0], qa[s][1], qa[s][2], qa[s][3], b2, b3);
                }
            }
            // ---- online softmax of query row g over the 16 positions (this thread: positions 2*t4, +1, +8, +9)
            float sv[4] = {s0[0] * p.scale_log2, s0[1] * p.scale_log2, s1[0] * p.scale_log2, s1[1] * p.scale_log2};
            const int pc[4] = {tpos + 2 * t4, tpos + 2 * t4 + 1, tpos + 8 + 2 * t4, tpos + 9 + 2 * t4};
#pragma unroll
            for (int i = 0; i < 4; ++i)
                if (pc[i] >= n_valid) sv[i] = -INFINITY;
            float mx = fmaxf(fmaxf(sv[0], sv[1]), fmaxf(sv[2], sv[3]));
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
            const float m_new = fmaxf(m_run, mx);  // finite: position tpos is valid
            const float corr = exp2f(m_run - m_new);
            float pe[4], psum = 0.f;
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                pe[i] = exp2f(sv[i] - m_new);
                psum += pe[i];
            }
            psum += __shfl_xor_sync(0xffffffffu, psum, 1);
            psum += __shfl_xor_sync(0xffffffffu, psum, 2);
            l_run = l_run * corr + psum;
            m_run = m_new;
            // P as the A operand of the second product: rows g use (positions 2t4, +1) and (+8, +9); rows g + 8 are zero
            const uint32_t pa0 = pack2_bf16(pe[0], pe[1]), pa2 = pack2_bf16(pe[2], pe[3]);
            // ---- O = O * corr + P V
            {
                // matrices for two n-tiles (16 values of d): (positions 0-7, d 0-7), (positions 8-15, d 0-7), (0-7, d 8-15), (8-15, d 8-15)
                const int r = row0 + (lane & 7) + ((lane >> 3) & 1) * 8, half = lane >> 4;
#pragma unroll
                for (int j = 0; j < NTILES; j += 2) {
                    uint32_t b0, b1, b2, b3;
                    ldsm_x4_trans(at_smem(vs) + tile_off<D>(r, j + half), b0, b1, b2, b3);
                    o[j][0] *= corr; o[j][1] *= corr; o[j + 1][0] *= corr; o[j + 1][1] *= corr;
                    mma_bf16(o[j], pa0, 0u, pa2, 0u, b0, b1);
                    mma_bf16(o[j + 1], pa0, 0u, pa2, 0u, b2, b3);
                }
            }
        }
        __syncthreads();  // every warp is done with this stage before it is refilled
        if (tile != tpu - 1 && gt != gt1 - 1) continue;

        // ---- this CTA's share of unit u is complete: merge the four warps (each saw a quarter of the positions of
        // every tile) through shared memory, half of the head dimension per round, rows < G only
        const int first_cta = u * tpu / R, last_cta = ((u + 1) * tpu - 1) / R;
        const int expected = last_cta - first_cta + 1, slot = static_cast<int>(blockIdx.x) - first_cta;
        const int64_t head0 = static_cast<int64_t>(u) * G;
        if (t4 == 0) {
            red_ml[(warp * 8 + g) * 2] = m_run;
            red_ml[(warp * 8 + g) * 2 + 1] = l_run;
        }
#pragma unroll
        for (int h = 0; h < 2; ++h) {
#pragma unroll
            for (int jj = 0; jj < HALF_NT; ++jj) {
                const int j = h * HALF_NT + jj;
                red_o[(warp * 8 + g) * (D / 2) + jj * 8 + 2 * t4] = o[j][0];
                red_o[(warp * 8 + g) * (D / 2) + jj * 8 + 2 * t4 + 1] = o[j][1];
            }
            __syncthreads();
            for (int i = tid; i < G * (D / 2); i += AT_THREADS) {
                const int r = i / (D / 2), dd = i % (D / 2), d = h * (D / 2) + dd;
                float mstar = -INFINITY;
#pragma unroll
                for (int w = 0; w < AT_WARPS; ++w) mstar = fmaxf(mstar, red_ml[(w * 8 + r) * 2]);
                float acc = 0.f, l = 0.f;
#pragma unroll
                for (int w = 0; w < AT_WARPS; ++w) {
                    const float mw = red_ml[(w * 8 + r) * 2];
                    const float f = mw == -INFINITY ? 0.f : exp2f(mw - mstar);
                    acc += red_o[(w * 8 + r) * (D / 2) + dd] * f;
                    l += red_ml[(w * 8 + r) * 2 + 1] * f;
                }
                if (expected == 1) {
                    p.out[(head0 + r) * D + d] = __float2bfloat16_rn(l > 0.f ? acc / l : 0.f);
                } else {
                    const int64_t ps = (static_cast<int64_t>(u) * p.kmax + slot) * G + r;
                    p.part_o[ps * D + d] = acc;
                    if (d == 0) {
                        p.part_ml[ps * 2] = mstar;
                        p.part_ml[ps * 2 + 1] = l;
                    }
                }
            }
            __syncthreads();
        }
        if (expected == 1) continue;
        // ---- the last of the CTAs that share unit u merges their partial results
        __threadfence();
        __syncthreads();
        if (tid == 0) {
            const int done = atomicAdd(&p.tickets[u], 1);
            s_last = done == expected - 1;
            if (s_last) p.tickets[u] = 0;  // ready for the next launch
        }
        __syncthreads();
        if (s_last) {
            __threadfence();
            // Weights of the partial results first (one parallel round of loads, kept in shared memory), then every
            // thread sums its outputs with independent loads: two memory round trips, not one per partial result.
            float* w_s = red_o;                      // [G][expected]
            float* m_s = w_s + 8 * AT_MAX_SPLITS;    // [G][expected]
            float* l_s = m_s + 8 * AT_MAX_SPLITS;    // [G]
            for (int i = tid; i < G * expected; i += AT_THREADS) {
                const int r = i / expected, sp = i % expected;
                const float2 ml = __ldcg(reinterpret_cast<const float2*>(p.part_ml) + (static_cast<int64_t>(u) * p.kmax + sp) * G + r);
                m_s[i] = ml.x;
                w_s[i] = ml.y;  // the sum, until the weight replaces it below
            }
            __syncthreads();
            if (tid < G) {
                float mstar = -INFINITY;
                for (int sp = 0; sp < expected; ++sp) mstar = fmaxf(mstar, m_s[tid * expected + sp]);
                float l = 0.f;
                for (int sp = 0; sp < expected; ++sp) {
                    const float ms = m_s[tid * expected + sp];
                    const float f = ms == -INFINITY ? 0.f : exp2f(ms - mstar);
                    l += w_s[tid * expected + sp] * f;
                    w_s[tid * expected + sp] = f;
                }
                l_s[tid] = l;
            }
            __syncthreads();
            for (int i = tid; i < G * D; i += AT_THREADS) {
                const int r = i / D, d = i % D;
                const float* po = p.part_o + (static_cast<int64_t>(u) * p.kmax * G + r) * D + d;
                float acc = 0.f;
#pragma unroll 8
                for (int sp = 0; sp < expected; ++sp) acc += __ldcg(po + static_cast<int64_t>(sp) * G * D) * w_s[r * expected + sp];
                const float l = l_s[r];
                p.out[(head0 + r) * D + d] = __float2bfloat16_rn(l > 0.f ? acc / l : 0.f);
            }
        }
        __syncthreads();  // red_* are free again
    }
    cp_async_wait<0>();
}

// CTAs of a launch: two per SM, never more than one per 64-position tile, and at most AT_SPLIT_CAP per unit: the partial
// results of a unit must stay within the merge buffers (AT_MAX_SPLITS - 2), and with one or two sequences a merge over
// more than sixteen partial results costs more than the shorter streams save (measured, 8 KV heads, context 2080:
// 15.0 -> 12.9 us at one sequence, 15.5 -> 13.6 us at two).
constexpr int AT_SPLIT_CAP = 16;
static_assert(AT_SPLIT_CAP <= AT_MAX_SPLITS - 2, "partial results of a unit");
static int attn_grid(int64_t units, int T) {
    const int64_t tiles = (T + AT_TILE - 1) / AT_TILE;
    int64_t g = 2LL * num_sms();
    if (g > units * tiles) g = units * tiles;
    if (g > units * AT_SPLIT_CAP) g = units * AT_SPLIT_CAP;
    return static_cast<int>(g < 1 ? 1 : g);
}
static int attn_kmax(int64_t units, int grid) { return static_cast<int>((grid + units - 1) / units + 2); }
constexpr int64_t AT_TICKET_UNITS = 16384;  // units that may be shared between CTAs: the ticket region is fixed, 64 KB

template <int D>
static int launch_attn(const AttnParams& p, int grid, unsigned flags, cudaStream_t st) {
    constexpr size_t smem = 16 * D * 2 + AT_STAGES * 2 * AT_TILE * D * 2 + AT_WARPS * 8 * (D / 2) * 4 + AT_WARPS * 8 * 2 * 4;
    static_assert(AT_WARPS * 8 * (D / 2) + AT_WARPS * 8 * 2 >= 2 * 8 * AT_MAX_SPLITS + 8, "the merge scratch must fit the warp-merge buffers");
    static PerDeviceOnce configured;
    const int dev = current_device();
    if (configured.needs(dev)) {
        WF_CUDA(cudaFuncSetAttribute(attn_decode_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
        configured.mark(dev);
    }
    cudaLaunchConfig_t lc = {};
    lc.gridDim = dim3(grid);
    lc.blockDim = dim3(AT_THREADS);
    lc.dynamicSmemBytes = smem;
    lc.stream = st;
    cudaLaunchAttribute attr[1];
    if (flags & WF_FLAG_PDL) {
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = 1;
        lc.attrs = attr;
        lc.numAttrs = 1;
    }
    WF_CUDA(cudaLaunchKernelEx(&lc, attn_decode_kernel<D>, p));
    return WF_OK;
}

}  // namespace wf

using namespace wf;

// workspace: [tickets: a fixed region of AT_TICKET_UNITS ints, so that launches of other shapes that share the workspace
// never put partial results where this shape keeps its tickets] [partial outputs] [partial maxima and sums]
extern "C" size_t wf_attn_decode_workspace_bytes(int64_t B, int nq, int nkv, int D, int T) {
    if (B <= 0 || nq <= 0 || nkv <= 0 || D <= 0 || T <= 0) return 0;
    const int64_t units = B * nkv;
    const int grid = attn_grid(units, T), kmax = attn_kmax(units, grid), G = nq / nkv;
    size_t bytes = static_cast<size_t>(AT_TICKET_UNITS) * sizeof(int);
    if (units <= AT_TICKET_UNITS) bytes += static_cast<size_t>(units) * kmax * G * (D + 2) * sizeof(float);
    return bytes;
}

extern "C" int wf_attn_decode_bf16(const void* q, const void* kcache, const void* vcache, const int64_t* pos, void* out, int64_t B,
                                   int nq, int nkv, int D, int T, float scale, void* workspace, size_t workspace_bytes, unsigned flags,
                                   void* stream) {
    WF_REQUIRE(q && kcache && vcache && out, "wf_attn_decode_bf16: null pointer");
    WF_REQUIRE(B > 0 && nq > 0 && nkv > 0 && T > 0 && B * nkv * ((T + AT_TILE - 1) / AT_TILE) < (1LL << 30),
               "wf_attn_decode_bf16: empty or oversized problem");
    WF_REQUIRE(nq % nkv == 0 && nq / nkv <= 8, "wf_attn_decode_bf16: query heads must be a multiple (at most 8) of the KV heads");
    WF_REQUIRE(D == 64 || D == 128, "wf_attn_decode_bf16: head dimension must be 64 or 128 (got %d)", D);
    WF_REQUIRE(reinterpret_cast<uintptr_t>(q) % 16 == 0 && reinterpret_cast<uintptr_t>(kcache) % 16 == 0 &&
                   reinterpret_cast<uintptr_t>(vcache) % 16 == 0,
               "wf_attn_decode_bf16: q and the caches must be 16-byte aligned");
    if (workspace_bytes < wf_attn_decode_workspace_bytes(B, nq, nkv, D, T) || !workspace)
        return fail(WF_E_SCRATCH, "wf_attn_decode_bf16: workspace of %zu bytes, need %zu", workspace_bytes,
                    wf_attn_decode_workspace_bytes(B, nq, nkv, D, T));
    WF_REQUIRE(reinterpret_cast<uintptr_t>(workspace) % 256 == 0, "wf_attn_decode_bf16: workspace must be 256-byte aligned");
    if (int rc = require_device()) return rc;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    AttnParams p;
    p.q = static_cast<const __nv_bfloat16*>(q);
    p.k = static_cast<const __nv_bfloat16*>(kcache);
    p.v = static_cast<const __nv_bfloat16*>(vcache);
    p.pos = pos;
    p.out = static_cast<__nv_bfloat16*>(out);
    p.nq = nq; p.nkv = nkv; p.T = T;
    p.units = static_cast<int>(B * nkv);
    const int grid = attn_grid(p.units, T);
    p.kmax = attn_kmax(p.units, grid);
    p.scale_log2 = scale * 1.4426950408889634f;
    uint8_t* ws = static_cast<uint8_t*>(workspace);
    p.tickets = reinterpret_cast<int*>(ws);
    p.part_o = reinterpret_cast<float*>(ws + static_cast<size_t>(AT_TICKET_UNITS) * sizeof(int));
    p.part_ml = p.part_o + static_cast<size_t>(p.units) * p.kmax * (nq / nkv) * D;
    p.unit_aligned = p.units > AT_TICKET_UNITS ? 1 : 0;
    return D == 64 ? launch_attn<64>(p, grid, flags, st) : launch_attn<128>(p, grid, flags, st);
}
