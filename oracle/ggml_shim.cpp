// C-ABI shim around BitNet.cpp's I2_S CPU routines.
//
// TEST INFRASTRUCTURE ONLY.  This file contains no reference code: it is compiled together with the reference's
//   packages/inference/extern/BitNet/src/ggml-bitnet-mad.cpp
// (read in place, never copied; only headers of its vendored ggml tree are on the include path) and exports plain-C
// entry points for the tests and the CPU-baseline leg of the benchmark.  The one ggml symbol that file links against,
// ggml_row_size, only feeds the byte count quantize_i2_s returns; it is supplied here for the I2_S type.
#include <cstddef>
#include <cstdint>

#include "ggml.h"  // found through -I<reference>/…/3rdparty/llama.cpp/ggml/include

#ifdef _OPENMP
#include <omp.h>
#endif

extern "C" {

// declared in the reference's ggml-quants.h; defined in its ggml-bitnet-mad.cpp
size_t quantize_i2_s(const float* src, void* dst, int64_t nrow, int64_t n_per_row, const float* quant_weights);
void ggml_vec_dot_i2_i8_s(int n, float* s, size_t bs, const void* vx, size_t bx, const void* vy, size_t by, int nrc);

size_t ggml_row_size(enum ggml_type type, int64_t ne) {
    (void)type;
    return static_cast<size_t>(ne);  // quantize_i2_s divides by 4 itself: 2 bits per weight
}

int ggml_ref_num_threads() {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

void ggml_ref_set_num_threads(int n) {
#ifdef _OPENMP
    if (n > 0) omp_set_num_threads(n);
#else
    (void)n;
#endif
}

// ggml-bitnet-mad.cpp:46-92: dst receives nrow * n_per_row / 4 bytes of codes followed by the fp32 scale
size_t ggml_ref_quantize_i2_s(const float* src, void* dst, int64_t nrow, int64_t n_per_row) {
    return quantize_i2_s(src, dst, nrow, n_per_row, nullptr);
}

// ggml-bitnet-mad.cpp:94: sum_k code[k] * a[k] of one packed row (the sum of a is NOT subtracted)
float ggml_ref_vec_dot(int n, const uint8_t* packed_row, const int8_t* act) {
    float s = 0.f;
    ggml_vec_dot_i2_i8_s(n, &s, 0, packed_row, 0, act, 0, 1);
    return s;
}

// the row loop of ggml's mul_mat over that routine, with its glue arithmetic (ggml.c:12491-12493):
// out[b, r] = (dot(row r, act b) - act_sum[b]) / act_scale[b] * w_scale
void ggml_ref_mul_mat(int rows, int K, int batch, float* out, const uint8_t* packed, const int8_t* act, const float* act_sums,
                      const float* act_scales, float w_scale) {
#pragma omp parallel for schedule(static)
    for (int r = 0; r < rows; ++r) {
        for (int b = 0; b < batch; ++b) {
            float s = 0.f;
            ggml_vec_dot_i2_i8_s(K, &s, 0, packed + static_cast<int64_t>(r) * (K / 4), 0, act + static_cast<int64_t>(b) * K, 0, 1);
            out[static_cast<int64_t>(b) * rows + r] = (s - act_sums[b]) / act_scales[b] * w_scale;
        }
    }
}
}
