// Contraction for large token counts (prefill): stand-alone activation
// quantization into the caller's workspace, then the integer contraction.
#include "wf_common.cuh"

int wf_check_linear_args(const char* who, const void* x, int x_dtype, int64_t ldx, const float* x_scale, const uint8_t* codes,
                         int layout, const void* bias, int bias_dtype, void* y, int y_dtype, int64_t ldy, int64_t M, int64_t N,
                         int64_t K);

using namespace wf;

static size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

extern "C" size_t wf_prefill_workspace_bytes(int64_t M, int64_t K) {
    if (M <= 0 || K <= 0) return 0;
    return align_up(static_cast<size_t>(M) * K, 256) + align_up(static_cast<size_t>(M) * 4, 256);
}

extern "C" int wf_bitlinear_prefill(const void* x, int x_dtype, int64_t ldx, const float* x_scale, const uint8_t* codes,
                                    int layout, const float* w_scale, float w_scale_host, const void* bias, int bias_dtype,
                                    void* y, int y_dtype, int64_t ldy, int32_t* acc_out, int64_t M, int64_t N, int64_t K,
                                    float eps, void* workspace, size_t workspace_bytes, unsigned flags, void* stream) {
    if (int rc = wf_check_linear_args("wf_bitlinear_prefill", x, x_dtype, ldx, x_scale, codes, layout, bias, bias_dtype, y,
                                      y_dtype, ldy, M, N, K))
        return rc;
    const int8_t* q = static_cast<const int8_t*>(x);
    const float* qs = x_scale;
    int64_t ldq = ldx;
    if (x_dtype != WF_I8) {
        WF_REQUIRE(workspace && reinterpret_cast<uintptr_t>(workspace) % 256 == 0, "wf_bitlinear_prefill: workspace must be 256-byte aligned");
        if (workspace_bytes < wf_prefill_workspace_bytes(M, K))
            return fail(WF_E_SCRATCH, "wf_bitlinear_prefill: workspace of %zu bytes, need %zu", workspace_bytes,
                        wf_prefill_workspace_bytes(M, K));
        int8_t* wq = static_cast<int8_t*>(workspace);
        float* ws = reinterpret_cast<float*>(static_cast<uint8_t*>(workspace) + align_up(static_cast<size_t>(M) * K, 256));
        if (int rc = wf_act_quant_i8(x, x_dtype, M, K, ldx, WF_ACT_PER_TOKEN, eps, wq, ws, nullptr, stream)) return rc;
        q = wq;
        qs = ws;
        ldq = K;
    }
    return wf_bitlinear_decode(q, WF_I8, ldq, qs, codes, layout, w_scale, w_scale_host, bias, bias_dtype, y, y_dtype, ldy,
                               acc_out, M, N, K, eps, flags, stream);
}
