// C-ABI shim around the reference's own CPU kernels.
//
// TEST INFRASTRUCTURE ONLY.  This file contains no reference code: it is
// compiled together with the reference's
//   packages/inference/extern/sglang-bitnet/sgl-kernel/csrc/bitnet/bitnet_gemv.cpp
// (read in place, never copied) and exports plain-C entry points so that the
// tests and the CPU-baseline leg of the benchmark can call the reference
// through ctypes.
#include <cstdint>
#include <exception>

#include "bitnet_gemv.h"  // found through -I<reference>/…/csrc/bitnet

#ifdef _OPENMP
#include <omp.h>
#endif

extern "C" {

int ref_num_threads() {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

// the OpenMP team size of the kernels below (a launcher may have exported OMP_NUM_THREADS=1)
void ref_set_num_threads(int n) {
#ifdef _OPENMP
    if (n > 0) omp_set_num_threads(n);
#else
    (void)n;
#endif
}

// bitnet_gemv.h:45-50
int ref_vec_dot_i2_i8(int n, float* result, const uint8_t* packed, const int8_t* act) {
    try {
        sgl_kernel::bitnet::bitnet_vec_dot_i2_i8(n, result, packed, act);
    } catch (const std::exception&) {
        return 1;
    }
    return 0;
}

// bitnet_gemv.h:64-73; output is laid out [M(out rows), N(batch)]
int ref_gemm_i2_i8(int M, int N, int K, float* out, const uint8_t* packed, const int8_t* act, float scale) {
    try {
        sgl_kernel::bitnet::bitnet_gemm_i2_i8(M, N, K, out, packed, act, scale);
    } catch (const std::exception&) {
        return 1;
    }
    return 0;
}

// the loop of bitnet_gemv_cpu (torch_extension_cpu.cpp:355-366): one dot product per output row
int ref_gemv_rows(int out_features, int K, float* out, const uint8_t* packed, const int8_t* act, float scale) {
    int err = 0;
#pragma omp parallel for
    for (int i = 0; i < out_features; ++i) {
        float r = 0.f;
        try {
            sgl_kernel::bitnet::bitnet_vec_dot_i2_i8(K, &r, packed + (int64_t)i * (K / 4), act);
        } catch (const std::exception&) {
            err = 1;
        }
        out[i] = r * scale;
    }
    return err;
}

// bitnet_gemv.h:83-88
void ref_quantize_activations_i8(int n, int8_t* out, const float* in, float* scale) {
    sgl_kernel::bitnet::quantize_activations_i8(n, out, in, scale);
}
}
