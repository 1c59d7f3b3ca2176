/*
 * wf_b200 — C ABI of the B200 (sm_100a) ternary BitLinear library.
 *
 * Every entry point returns 0 on success or a WF_E_* code; wf_last_error()
 * gives the message of the calling thread's last failure.  Nothing throws and
 * nothing exits.  All pointers are device pointers unless a comment says
 * "host".  The caller owns every buffer; the library allocates nothing.
 * `stream` is a cudaStream_t passed as void* (NULL = the default stream).
 * Calls are asynchronous on that stream.  There is no CPU fallback: on a machine
 * without an sm_100 device every compute entry point fails with WF_E_DEVICE.
 *
 * Each declaration cites the interface of the reference project that it
 * replaces (paths inside that project).
 */
#ifndef WF_B200_H
#define WF_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---- status codes ---- */
#define WF_OK 0
#define WF_E_ARG 1       /* bad argument: null pointer, size, alignment, unsupported dtype */
#define WF_E_DEVICE 2    /* no usable sm_100 device / CUDA runtime error */
#define WF_E_SCRATCH 3   /* scratch buffer too small */
#define WF_E_LIMIT 4     /* size beyond a documented maximum */

/* ---- element types of activations / weights / outputs ---- */
#define WF_F32 0
#define WF_F16 1
#define WF_BF16 2
#define WF_I8 3 /* activations already quantized to int8 */

/* ---- layouts of packed 2-bit weights (code = w + 1, 4 per byte, row-major [N, K/4]) ---- */
#define WF_LAYOUT_WF16 0    /* this library's layout: per 32-bit word, byte b bit-pair j = weight 16*word + 4*j + b; K % 64 == 0 */
#define WF_LAYOUT_I2S 1     /* 128-weight blocks of 32 bytes: byte j bits 7:6,5:4,3:2,1:0 = weights j, j+32, j+64, j+96; K % 128 == 0 */
#define WF_LAYOUT_SEQ_LSB 2 /* byte j = weights 4j..4j+3 at shifts 0,2,4,6 (conversion only: the kernels do not consume it) */
#define WF_LAYOUT_SEQ_MSB 3 /* byte j = weights 4j..4j+3 at shifts 6,4,2,0 (conversion only) */
#define WF_LAYOUT_HF 4      /* [N/4, K] bytes: byte (r,c) = rows r, r+N/4, r+2N/4, r+3N/4 at shifts 0,2,4,6 (conversion source only) */

/* ---- ternarization modes of wf_pack_ternary ---- */
#define WF_PACK_FP32 0      /* scale = mean|w| in fp32, codes = clamp(rint(w / scale)) */
#define WF_PACK_CAST_BF16 1 /* cast to bf16 first, every intermediate rounded to bf16 */
#define WF_PACK_CAST_F16 2  /* cast to f16 first, every intermediate rounded to f16 */

/* ---- activation quantization modes of wf_act_quant_i8 ---- */
#define WF_ACT_PER_TOKEN 0  /* per row absmax, arithmetic in the element type of x */
#define WF_ACT_PER_TENSOR 1 /* one absmax for the whole tensor, fp32, scale = max/127 returned */

/* ---- fused input modes of a grouped decode problem (wf_problem.x_mode) ---- */
#define WF_X_PLAIN 0
#define WF_X_SILU 1
#define WF_X_RELU2 2
#define WF_X_NORM 3

/* ---- launch flags of the contraction entry points ---- */
#define WF_FLAG_PDL 1u /* launch with programmatic stream serialization: the kernel streams its
                          first weights before it waits for the previous kernel of the stream */
#define WF_FLAG_X_READY 2u /* with WF_FLAG_PDL, grouped streaming launches only: the caller states that x was NOT
                              written by the previous kernel of the stream (independent layers, experts, replicas).
                              The kernel then reads x without waiting and only its stores wait for that kernel.
                              The tensor-core contraction takes it together with WF_FLAG_WS_READY (below); the other
                              forms ignore it.  No counterpart in the reference (its CPU operators are synchronous
                              calls). */

#define WF_FLAG_WS_READY 16u /* wf_bitlinear_prefill(_batched): the workspace already holds the quantized tokens of this x
                                (wf_prefill_quantize earlier in the stream); x is not read.  One quantization then serves
                                every projection of the same tokens (q/k/v, gate/up), as the shared act-quant of
                                bitnet_qkv_forward_cpu / bitnet_mlp_forward_cpu does
                                (packages/inference/extern/sglang-bitnet/sgl-kernel/csrc/cpu/bitnet_fused_layer.cpp:150-375).
                                With WF_FLAG_X_READY in addition (only directly behind another wf_bitlinear_prefill(_batched)
                                launch in the stream, flagged or not) the caller states that the workspace was filled, and y
                                / acc_out last touched, before the most recent UNFLAGGED one of those launches -- in
                                practice: the quantizations go first, then one contraction without the flag, then the
                                flagged ones, each with a workspace and an output of its own.  An unflagged contraction
                                lets the launches behind it start only once everything ahead of it has completed; a flagged
                                one waits for nothing before its loads and stores, so it fills the SMs that the tail of the
                                previous contraction leaves idle.  Its grid still ends after its predecessor. */

#define WF_FLAG_PREFILL_PAIR 4u   /* wf_bitlinear_prefill, more than 64 tokens: use the form in which two CTAs (a cluster of two
                                     SMs, tcgen05 cta_group::2) share each 256-row x 192-token tile (half the token bytes from
                                     L2 per multiply-add; measured slower than the default on B200) */
#define WF_FLAG_PREFILL_SINGLE 8u /* ... the form with one CTA per 128-row x 128-token tile (the default) */

int wf_version(void);
const char* wf_last_error(void);

/* Returns WF_OK when the current CUDA device can run this library (compute capability 10.x). */
int wf_device_check(void);

/*
 * Measurement aid, no counterpart in the reference: the rate of the int8 tensor-core instruction on the current
 * device.  Every SM issues 4 * iters tcgen05.mma.kind::i8 (M = 128, N = n, K = 32) on operands resident in shared
 * memory; *tops_out receives 2 * 128 * n * 32 operations per instruction over the measured time, summed over the
 * SMs (the measured denominator of the contraction's roofline), *ns_per_mma_out (nullable) the time per instruction
 * of one SM.  Synchronizes the device; runs on the default stream.
 */
int wf_probe_i8_mma(int n, int iters, double* tops_out, double* ns_per_mma_out);

/*
 * Absmean ternarization + 2-bit packing of a weight matrix into WF_LAYOUT_WF16.
 * Replaces: ternary_weight_quantization_no_scale (packages/training/src/wrinklefree/quantization/weight_quant.py:35-56),
 *           BitLinear.weight_quant for the cast-first modes (packages/training/src/wrinklefree/models/bitlinear.py:46-64,103),
 *           pack_ternary_sglkernel (packages/inference/scripts/convert_to_sglkernel.py:51-123).
 * w: [N, K] row-major with row stride ldw elements, type w_dtype (WF_F32/WF_F16/WF_BF16).
 * codes_out: [N, K/4] bytes.  scale_out: 2 floats: [0] the dequantization multiplier
 * (mean|w| for WF_PACK_FP32; the rounded 1/scale of the forward for the cast-first
 * modes), [1] the quantization multiplier actually used.  K % 64 == 0.
 * scratch: at least wf_pack_scratch_bytes(N, K) bytes of device memory, 16-byte aligned.
 * The sum of |w| is carried in fp64 in a fixed order: results are deterministic.
 */
size_t wf_pack_scratch_bytes(int64_t N, int64_t K);
int wf_pack_ternary(const void* w, int w_dtype, int64_t N, int64_t K, int64_t ldw, int mode, float eps,
                    uint8_t* codes_out, float* scale_out, void* scratch, size_t scratch_bytes, void* stream);

/*
 * wf_pack_ternary for callers that must not allocate: same arguments without the scratch pair.
 * This entry point has no counterpart in the reference.  It is for hosts where device allocation is
 * off-limits at the point of packing (a serving process whose memory pool owns the GPU and forbids
 * cudaMalloc in layer code, or a latency-critical thread that cannot take an allocation's implicit device
 * synchronisation).  The scratch is a fixed array inside the library image on every GPU that loads it
 * (wf_pack_noalloc_scratch_bytes() = 9472 bytes, held until exit); the call allocates and frees nothing.
 * Limit: N * K <= WF_PACK_NOALLOC_MAX_WEIGHTS, larger matrices are refused with WF_E_LIMIT.
 * The first call on a device resolves the array's device address: make it outside any stream capture.
 * All calls on a device share the array, so calls that overlap on the GPU race; every launch overwrites
 * what it reads, nothing needs clearing between calls.  Results are identical to wf_pack_ternary's.
 */
#define WF_PACK_NOALLOC_MAX_WEIGHTS ((int64_t)1 << 28)
size_t wf_pack_noalloc_scratch_bytes(void);
int wf_pack_ternary_noalloc(const void* w, int w_dtype, int64_t N, int64_t K, int64_t ldw, int mode, float eps,
                            uint8_t* codes_out, float* scale_out, void* stream);

/*
 * Layout conversion of already-ternary packed weights into dst_layout (any row-major layout: WF16, I2S, SEQ_LSB, SEQ_MSB).
 * Replaces the Python packing loops: _pack_ternary_weights (packages/inference/src/wrinklefree_inference/cache/bitnet_converter.py:26-77),
 * repack_hf_weights / pack_weights (packages/inference/src/wrinklefree_inference/kernels/native.py:181-241),
 * pack_ternary_weights (packages/inference/src/wrinklefree_inference/kernels/bitnet_patch.py:81-112).
 * N, K are the logical weight dimensions; src holds N*K/4 bytes in src_layout.
 */
int wf_repack(const uint8_t* src, int src_layout, uint8_t* dst, int dst_layout, int64_t N, int64_t K, void* stream);

/*
 * The max-abs quantizers of the inference side, on the GPU: scale_out[0] = max|w| and 2-bit codes written
 * straight into dst_layout (any row-major layout).  scale_out must hold 2 floats (the second is scratch).
 * WF_MAXABS_HALF replaces quantize_to_bitnet
 *   (packages/inference/src/wrinklefree_inference/sglang_backend/bitnet_quantization.py:69-109): a maximum below
 *   1e-6 counts as 1, codes +1 / -1 where w / max is above 0.5 / below -0.5, else 0; its bytes are WF_LAYOUT_SEQ_MSB.
 * WF_MAXABS_SIGN replaces quantize_i2_s (packages/inference/extern/BitNet/src/ggml-bitnet-mad.cpp:46-92): codes by
 *   the sign of w, 0 where |w| < 1e-6; its bytes are WF_LAYOUT_I2S (the scale that file appends after the data is
 *   returned in scale_out instead).
 */
#define WF_MAXABS_HALF 0
#define WF_MAXABS_SIGN 1
int wf_quantize_maxabs(const void* w, int w_dtype, int64_t N, int64_t K, int64_t ldw, int rule, int dst_layout,
                       uint8_t* codes_out, float* scale_out, void* stream);

/* Packs int8 ternary values {-1,0,1} [N,K] into `layout` (any row-major layout); unpacks the other way (any layout). */
int wf_pack_codes(const int8_t* ternary, uint8_t* dst, int layout, int64_t N, int64_t K, void* stream);
int wf_unpack_codes(const uint8_t* src, int layout, int8_t* ternary, int64_t N, int64_t K, void* stream);

/*
 * Activation quantization to int8.
 * Replaces: BitLinear.activation_quant (packages/training/src/wrinklefree/models/bitlinear.py:66-84) for WF_ACT_PER_TOKEN,
 *           quantize_activations_i8 / bitnet_quantize_activations_cpu
 *           (packages/inference/extern/sglang-bitnet/sgl-kernel/csrc/bitnet/bitnet_gemv.cpp:880-1135,
 *            .../csrc/cpu/torch_extension_cpu.cpp:409-427) for WF_ACT_PER_TENSOR.
 * x: [M, K] row stride ldx elements.  q: [M, K] int8 contiguous.
 * WF_ACT_PER_TOKEN: scale[m] = the multiplier rnd(rnd(1/max(absmax,eps))*127) in the arithmetic of x's type
 *   (the value the reference divides by to dequantize); rowsum[m] (nullable) = sum_k q[m,k].
 * WF_ACT_PER_TENSOR: x must be WF_F32; scale[0] = max/127 (max < 1e-6 counts as 1); rowsum as above.
 *   Rounding is to nearest even everywhere.
 */
int wf_act_quant_i8(const void* x, int x_dtype, int64_t M, int64_t K, int64_t ldx, int mode, float eps, int8_t* q,
                    float* scale, int32_t* rowsum, void* stream);

/*
 * y[m, n] = (float(acc[m,n]) * inv_sx[m]) * s_w (+ bias[n]),  acc[m,n] = sum_k q[m,k] * w[n,k]  (int32, exact).
 *
 * wf_bitlinear_decode: fused per-token activation quantization + contraction for small token counts
 * (decode); any M is accepted, the weights are re-read once per group of tokens that fits in shared memory.
 * wf_bitlinear_prefill: the tensor-core (tcgen05) contraction for large token counts; needs
 * workspace of wf_prefill_workspace_bytes(M, K) bytes when x is not WF_I8.
 *
 * Replace: BitLinear.forward at lambda = 1 (packages/training/src/wrinklefree/models/bitlinear.py:86-113),
 *          bitnet_gemv_cpu / bitnet_gemm_cpu (packages/inference/extern/sglang-bitnet/sgl-kernel/csrc/cpu/torch_extension_cpu.cpp:331-407),
 *          bitnet_vec_dot_i2_i8 / bitnet_gemm_i2_i8 (.../csrc/bitnet/bitnet_gemv.cpp:325-874),
 *          BitNetLinearMethod.apply (packages/inference/extern/sglang-bitnet/python/sglang/srt/layers/quantization/bitnet.py:205-255).
 *
 * x: [M, K] of x_dtype, row stride ldx elements.  With WF_I8, x is int8 [M, K]; x_scale (nullable, [M])
 *    holds the per-token multipliers (inv_sx = 1/x_scale[m], 1 when null) and x_rowsum is ignored.
 *    Otherwise x_scale must be null and inv_sx[m] = 1/scale[m] with scale as in wf_act_quant_i8 per token.
 * codes: [N, K/4] in `layout` (WF16 or I2S).
 * w_scale: device pointer to s_w (nullable: then s_w = w_scale_host).
 * bias: nullable, [N] of bias_dtype.   y: [M, N] of y_dtype, row stride ldy elements.
 * acc_out: nullable, int32 [M, N] contiguous: the raw integer accumulators, for bit-exact checks.
 */
int wf_bitlinear_decode(const void* x, int x_dtype, int64_t ldx, const float* x_scale, const uint8_t* codes,
                        int layout, const float* w_scale, float w_scale_host, const void* bias, int bias_dtype,
                        void* y, int y_dtype, int64_t ldy, int32_t* acc_out, int64_t M, int64_t N, int64_t K,
                        float eps, unsigned flags, void* stream);

/*
 * Grouped form of wf_bitlinear_decode: P independent problems (for example the q/k/v or gate/up
 * projections of one layer, or a stack of layers) run as ONE persistent kernel, so that weight
 * streaming of one problem overlaps everything else of the others.  Replaces the per-projection loops of
 * bitnet_qkv_forward_cpu / bitnet_mlp_forward_cpu
 * (packages/inference/extern/sglang-bitnet/sgl-kernel/csrc/cpu/bitnet_fused_layer.cpp:150-375).
 *
 * Fields have the meaning of the wf_bitlinear_decode arguments of the same name.  All problems of a group
 * share x_dtype.  The fields starting with an underscore are filled by wf_bitlinear_decode_plan.
 * The struct is 576 bytes and both copies must start on a 64-byte boundary (it embeds TMA descriptors).
 * Use: fill a host array, call wf_bitlinear_decode_plan on it, copy it unchanged to device memory
 * (it must stay there while the kernel runs; it may be reused for any number of launches), then call
 * wf_bitlinear_decode_grouped with both copies.
 */
#if defined(__GNUC__) || defined(__clang__) || defined(__CUDACC__)
#define WF_ALIGN64 __attribute__((aligned(64)))
#else
#define WF_ALIGN64 __declspec(align(64))
#endif
typedef struct WF_ALIGN64 wf_problem {
    const void* x;
    const float* x_scale;
    const uint8_t* codes;
    const float* w_scale;
    const void* bias;
    void* y;
    int32_t* acc_out;
    int64_t ldx, ldy;
    int32_t M, N, K;
    int32_t x_dtype, y_dtype, bias_dtype, layout;
    float w_scale_host, eps;
    int32_t _item_begin, _row_items, _chunks, _kb_full, _tail_bytes; /* 128 bytes up to here */
    int32_t _kb_seg, _ksegs; /* K is streamed in _ksegs segments of _kb_seg 512-weight blocks */
    /* Fused input (bf16 x only; zero-initialise for a plain projection).  The activations the projection quantizes are
     * computed on the fly, with the arithmetic of the unfused kernels of this library:
     *   WF_X_SILU / WF_X_RELU2: act(x) * x2, x = gate and x2 = up of an MLP (wf_act_mul_bf16) - replaces the activation
     *     in front of down_proj (packages/training/src/wrinklefree/models/ffn.py:74-87; bitnet_mlp_forward_cpu fuses it the
     *     same way, packages/inference/extern/sglang-bitnet/sgl-kernel/csrc/cpu/bitnet_fused_layer.cpp:150-375);
     *   WF_X_NORM: h = x (+ x2), then h * rsqrt(mean(h^2) + norm_eps) * norm_w (wf_add_rmsnorm_bf16) - the residual add and
     *     RMSNorm in front of q/k/v or gate/up (the A100 stack fuses the quantization into its norm,
     *     packages/inference/extern/BitNet/gpu/model.py:54-76); h_out (nullable) receives h, written once per launch.
     * x2 and h_out have the row stride of x. */
    const void* x2;
    const void* norm_w;
    void* h_out;
    int32_t x_mode;
    float norm_eps;
    /* Optional: a range of global memory (typically the packed weights of the NEXT launch of the stream) that this
     * launch asks the L2 cache to fetch while it runs (non-multicast cp.async.bulk.prefetch.L2, issued at kernel entry,
     * spread over the CTAs).  A decode step at small batch is a chain of short, latency-bound launches: with the next
     * weights on their way to L2 meanwhile, the HBM transfer overlaps the chain instead of adding to it.
     * prefetch_bytes must be a multiple of 16, prefetch 16-byte aligned; 0 / NULL: none. */
    const void* prefetch;
    int64_t prefetch_bytes;
    /* Optional: the exchange of a row-parallel projection fused into this launch.  A device pointer obtained from
     * wf_ar_xchg: besides writing y, the launch pushes its partial output into every rank's exchange buffer and
     * reports the delivered elements; wf_ar_reduce_add_rmsnorm on every rank then sums the partial outputs (see there).  y must be a
     * contiguous 16-bit tensor (ldy == N, N even) of at most the exchange's max_bytes; at most one problem of a launch
     * sets xchg.  NULL: none. */
    const void* xchg;
    uint64_t _tmap_main[16]; /* TMA descriptor: [K/512 blocks][N rows][128 bytes] view of codes, box of _kb_seg blocks */
    uint64_t _tmap_last[16]; /* the same view with the (shorter) box of the last segment */
    uint64_t _tmap_tail[16]; /* TMA descriptor of the last, partial 128-byte column block (if any) */
} wf_problem;

int wf_bitlinear_decode_plan(wf_problem* host_problems, int P);
int wf_bitlinear_decode_grouped(const wf_problem* dev_problems, const wf_problem* host_problems, int P, unsigned flags,
                                void* stream);

/* Last device-side status of the decode kernels on the current device: 0, or WF_E_LIMIT when a bounded
 * wait inside a kernel ran out (the kernel then finished without hanging; its outputs are invalid).
 * Synchronizes the device. */
int wf_device_status(void);

size_t wf_prefill_workspace_bytes(int64_t M, int64_t K);
int wf_bitlinear_prefill(const void* x, int x_dtype, int64_t ldx, const float* x_scale, const uint8_t* codes,
                         int layout, const float* w_scale, float w_scale_host, const void* bias, int bias_dtype,
                         void* y, int y_dtype, int64_t ldy, int32_t* acc_out, int64_t M, int64_t N, int64_t K,
                         float eps, void* workspace, size_t workspace_bytes, unsigned flags, void* stream);

/*
 * `batch` independent layers of one shape in one launch of the tensor-core contraction (a stack of layers, the
 * experts of a mixture, or the same projection of several model replicas).  Rows are stacked: x is
 * [batch * M, K] (row stride ldx), codes [batch * N, K/4], y [batch * M, N] (row stride ldy); layer z multiplies
 * tokens z*M .. z*M+M-1 with weight rows z*N .. z*N+N-1 and uses the scale w_scale[z * w_scale_stride].
 * acc_out (nullable) is [batch * M, N].  workspace: wf_prefill_workspace_bytes(batch * M, K) bytes.
 * Replaces the per-layer loop over bitnet_gemm_cpu
 * (packages/inference/extern/sglang-bitnet/sgl-kernel/csrc/cpu/torch_extension_cpu.cpp:370-407).
 */
int wf_bitlinear_prefill_batched(const void* x, int x_dtype, int64_t ldx, const uint8_t* codes, int layout,
                                 const float* w_scale, int64_t w_scale_stride, void* y, int y_dtype, int64_t ldy,
                                 int32_t* acc_out, int64_t batch, int64_t M, int64_t N, int64_t K, float eps,
                                 void* workspace, size_t workspace_bytes, unsigned flags, void* stream);

/* The quantization step of wf_bitlinear_prefill(_batched) on its own: per-token absmax int8 codes, scales and row sums
 * of x [M, K] (M = batch * tokens for a batched call) into `workspace` (wf_prefill_workspace_bytes(M, K) bytes), for
 * later calls with WF_FLAG_WS_READY on the same workspace.  Same arithmetic as wf_act_quant_i8 in per-token mode
 * (quantize_activations_i8, packages/inference/extern/sglang-bitnet/sgl-kernel/csrc/bitnet/bitnet_gemv.cpp).
 * flags: WF_FLAG_X_READY -- the caller states that no kernel that may still be running (the previous one of the stream
 * and, while those were launched with this flag too, the ones before it) writes x or uses the workspace: the kernel
 * starts at once instead of behind its predecessor (its grid still ends after it). */
int wf_prefill_quantize(const void* x, int x_dtype, int64_t ldx, int64_t M, int64_t K, float eps, void* workspace,
                        size_t workspace_bytes, unsigned flags, void* stream);

/*
 * Fused elementwise kernels around the projections of a decoder layer (bf16 tensors, contiguous rows).
 * They replace operator chains of the callers of BitLinear in the reference model
 * (packages/training/src/wrinklefree/models/subln.py / transformer.py:80-117 for residual + RMSNorm,
 *  attention.py:14-64 for RoPE, ffn.py:51-87 for the gate activation) in the decode step.
 * wf_add_rmsnorm_bf16: h[M,K] += delta (nullable), y = h * rsqrt(mean(h^2) + eps) * weight[K].
 * wf_rope_kv_bf16:     rotates q [B, nq*D] in place and k [B, nkv*D] at position *pos (device scalar; the caller keeps it below T, the
 *                      kernel only reduces it modulo T so that a stray value cannot leave the tables),
 *                      writes the rotated k and v into the caches [B, nkv, T, D]; cos/sin are fp32 [T, D/2].
 * wf_act_mul_bf16:     out = act(gate) * up over n elements; mode 0 = SiLU, 1 = ReLU^2.
 * flags: WF_FLAG_PDL chains the kernel to its neighbours in the stream with a programmatic dependency (each of
 * these kernels lets its successor start at once and waits for its predecessor before it touches a tensor).
 */
int wf_add_rmsnorm_bf16(void* h, const void* delta, const void* weight, void* y, int64_t M, int64_t K, float eps, unsigned flags,
                        void* stream);
int wf_rope_kv_bf16(void* q, const void* k, const void* v, const float* cos, const float* sin, const int64_t* pos, void* kcache,
                    void* vcache, int64_t B, int nq, int nkv, int D, int T, unsigned flags, void* stream);
int wf_act_mul_bf16(const void* gate, const void* up, void* out, int64_t n, int mode, unsigned flags, void* stream);
/*
 * The same two kernels with the per-token int8 quantization of the projection that follows fused in (the reference's
 * fused CPU layer shares one activation quantization between gate and up and the A100 stack quantizes inside its norm:
 * sgl-kernel/csrc/cpu/bitnet_fused_layer.cpp:150-375, BitNet/gpu/model.py:54-76): q [M, K] int8 and q_scale [M] receive
 * what wf_act_quant_i8(WF_ACT_PER_TOKEN, quant_eps) would produce from the bf16 result, bit for bit; the bf16 result
 * itself is written only when y / out is not NULL.  Rows of a multiple of 8 elements, at most 16384.
 */
int wf_add_rmsnorm_quant_bf16(void* h, const void* delta, const void* weight, void* y, int8_t* q, float* q_scale, int64_t M,
                              int64_t K, float eps, float quant_eps, unsigned flags, void* stream);
int wf_act_mul_quant_bf16(const void* gate, const void* up, void* out, int8_t* q, float* q_scale, int64_t M, int64_t I, int mode,
                          float quant_eps, unsigned flags, void* stream);

/*
 * Decode-step attention over the bf16 KV cache (one new token per sequence, grouped-query heads): for every query head
 * out[b, h, :] = softmax_t(scale * q[b, h, :] . K[b, kv(h), t, :]) V[b, kv(h), t, :] over the valid positions t.
 * Replaces, for the decode step, the attention core of the reference model
 * (packages/training/src/wrinklefree/models/attention.py:186-208: repeat_kv, QK^T, fp32 softmax, PV) on the layout of a
 * KV cache (packages/inference/src/wrinklefree_inference/kv_cache/kv_cache.py:96-370 keeps one; the reference model itself
 * recomputes the prompt every step).
 * q: [B, nq * D] bf16 (already rotated); kcache / vcache: [B, nkv, T, D] bf16; out: [B, nq * D] bf16.
 * pos: device scalar, positions 0 .. *pos are valid (nullable: all T positions).  nq % nkv == 0, nq / nkv <= 8, D = 64 or 128.
 * Keys and values are read once per step for the whole group of query heads; persistent CTAs share the tiles of all
 * (sequence, KV head) pairs evenly and merge shared pairs in the same launch.  workspace: wf_attn_decode_workspace_bytes(...) bytes, 256-byte aligned
 * (merge tickets and partial results), ZERO before its first use (every launch leaves its tickets zero again); it may
 * be shared by the launches of one stream, also of different shapes.  flags: WF_FLAG_PDL.
 */
size_t wf_attn_decode_workspace_bytes(int64_t B, int nq, int nkv, int D, int T);
int wf_attn_decode_bf16(const void* q, const void* kcache, const void* vcache, const int64_t* pos, void* out, int64_t B, int nq,
                        int nkv, int D, int T, float scale, void* workspace, size_t workspace_bytes, unsigned flags, void* stream);

/*
 * Dense bf16 linear layer: y[M, N] = x[M, K] . w[N, K]^T, bf16 operands (row strides ldx, ldw in elements, multiples
 * of 8; x and w 16-byte aligned; K a multiple of 8), fp32 accumulation on the tensor cores, y of y_dtype (WF_F32 /
 * WF_BF16 / WF_F16, row stride ldy).  It is the output head of the ternary decoder, the one matrix the reference keeps
 * in full precision (nn.Linear lm_head of BitNetLlama, packages/training/src/wrinklefree/models/llama.py:53,140; F.linear in
 * the serving runtime): one pass over w serves up to 256 tokens.  Takes WF_FLAG_PDL.
 */
int wf_linear_bf16(const void* x, int64_t ldx, const void* w, int64_t ldw, void* y, int y_dtype, int64_t ldy, int64_t M,
                   int64_t N, int64_t K, unsigned flags, void* stream);

/*
 * One-shot all-reduce (sum) over peer memory for the small tensors that follow a row-parallel projection in the
 * decode step; one process per GPU on one node.  It stands where the reference's tensor-parallel layers call the
 * library all-reduce after o_proj / down_proj (sglang/srt/layers/linear.py:1419-1420); larger tensors stay on NCCL.
 * Set-up, once per process group: every rank calls wf_ar_init (allocates its exchange buffer of 4 KiB + 2 * max_bytes
 * and returns a CUDA IPC handle of wf_ar_handle_bytes() bytes), the ranks exchange the handles by any means, and every
 * rank calls wf_ar_connect with all of them in rank order.  wf_ar_allreduce(in, out, n elements, dtype) may run in
 * place, must be called by every rank with the same n and dtype in the same order, sums in rank order in fp32 (all
 * ranks obtain identical bits) and takes WF_FLAG_PDL.  Its waits for the peers are bounded (about 0.1 s); a wait that
 * ran out is reported by wf_ar_status (WF_E_LIMIT) and leaves `out` undefined.
 * After such a report the ranks no longer agree on the step: wf_ar_step reads this rank's count of completed
 * all-reduces, and wf_ar_set_step (on every rank, with one common value above every rank's count, e.g. their maximum
 * + 2, between two host-side barriers and with no all-reduce in flight) puts the group back in step.
 */
/* The device-side descriptor of an exchange (filled by wf_ar_connect inside the exchange buffer). */
typedef struct wf_xchg {
    int32_t world, rank;
    uint64_t slot_bytes; /* capacity of one (slot, source) region = max_bytes of wf_ar_init */
    uint64_t push_off;   /* offset of the push regions inside every rank's buffer */
    void* peer[8];       /* every rank's buffer, as seen from this rank */
} wf_xchg;

int wf_ar_handle_bytes(void);
int wf_ar_init(int world, int rank, size_t max_bytes, void** ctx_out, unsigned char* handle_out);
int wf_ar_connect(void* ctx, const unsigned char* handles);
int wf_ar_allreduce(void* ctx, const void* in, void* out, int64_t n, int dtype, unsigned flags, void* stream);
int wf_ar_status(void* ctx, int* out);
int wf_ar_step(void* ctx, unsigned* out);
int wf_ar_set_step(void* ctx, unsigned step);
/*
 * The exchange fused into the row-parallel projection (the reference sums after o_proj / down_proj with a library
 * all-reduce, sglang/srt/layers/linear.py:1419-1420; its custom all-reduce pushes and polls in the same way,
 * sgl-kernel/csrc/allreduce/custom_all_reduce.cuh:203-260).  wf_ar_xchg returns the device pointer to put into
 * wf_problem.xchg of the projection's grouped launch.  wf_ar_reduce_add_rmsnorm is the consumer, on every rank, after that
 * launch in the same stream: it waits (bounded, about 0.2 s, then WF_E_LIMIT through wf_ar_status) until every rank
 * has pushed this step, forms delta = the sum of the partial outputs in rank order in fp32, rounded to bf16 (the bits
 * of wf_ar_allreduce on the same partial outputs), and continues as wf_add_rmsnorm_bf16(h, delta, weight, y): h += delta,
 * y = rmsnorm(h) * weight.  M x K bf16, K a multiple of 8 and at most 16384, M * K * 2 <= max_bytes.  Takes WF_FLAG_PDL.
 */
int wf_ar_xchg(void* ctx, const void** dev_desc_out);
int wf_ar_reduce_add_rmsnorm(void* ctx, void* h, const void* weight, void* y, int64_t M, int64_t K, float eps, unsigned flags,
                             void* stream);
/* ... with the per-token int8 quantization of the projections that follow fused in, as wf_add_rmsnorm_quant_bf16 (y may be NULL) */
int wf_ar_reduce_add_rmsnorm_quant(void* ctx, void* h, const void* weight, void* y, int8_t* q, float* q_scale, int64_t M, int64_t K,
                                   float eps, float quant_eps, unsigned flags, void* stream);
int wf_ar_destroy(void* ctx);

#ifdef __cplusplus
}
#endif
#endif /* WF_B200_H */
