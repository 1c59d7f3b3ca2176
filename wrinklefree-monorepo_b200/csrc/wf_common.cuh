// Shared helpers of the wf_b200 CUDA sources: error reporting, element-type
// conversion, the rounding rules of the reference's quantizers.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <cstdarg>
#include <cstdio>

#include "../../include/wf_b200.h"

namespace wf {

// ---- last-error string of the calling thread ----
char* err_buf();
int fail(int code, const char* fmt, ...);
int cuda_fail(cudaError_t e, const char* what);

#define WF_CUDA(call)                                        \
    do {                                                     \
        cudaError_t _e = (call);                             \
        if (_e != cudaSuccess) return ::wf::cuda_fail(_e, #call); \
    } while (0)

#define WF_REQUIRE(cond, ...)                          \
    do {                                               \
        if (!(cond)) return ::wf::fail(WF_E_ARG, __VA_ARGS__); \
    } while (0)

int require_device();  // WF_OK when the current device is compute capability 10.x

// Per-device facts, keyed by device index (a process, and a single host thread, may drive several GPUs).
constexpr int WF_MAX_DEVICES = 64;
int current_device();   // index of the current device, or -1
int num_sms();          // multiprocessors of the current device (148 when the query fails)

// One-time per-device set-up of a kernel (cudaFuncSetAttribute is a per-device setting): `done` is a table with
// one flag per device index; returns true when the caller still has to configure the current device.
struct PerDeviceOnce {
    unsigned char done[WF_MAX_DEVICES] = {};
    bool needs(int dev) const { return dev < 0 || dev >= WF_MAX_DEVICES || !done[dev]; }
    void mark(int dev) { if (dev >= 0 && dev < WF_MAX_DEVICES) done[dev] = 1; }
};

inline size_t dtype_size(int dt) { return dt == WF_F32 ? 4 : (dt == WF_I8 ? 1 : 2); }
inline bool is_float_dtype(int dt) { return dt == WF_F32 || dt == WF_F16 || dt == WF_BF16; }

// ---- rounding to the arithmetic type of the reference's elementwise ops ----
// MODE: WF_F32 identity, WF_BF16 / WF_F16 round-to-nearest-even to that type.
template <int MODE>
__device__ __forceinline__ float rnd(float v) {
    if constexpr (MODE == WF_BF16) return __bfloat162float(__float2bfloat16_rn(v));
    if constexpr (MODE == WF_F16) return __half2float(__float2half_rn(v));
    return v;
}

// The quantization multiplier of one token: torch evaluates `127.0 / t` as
// `t.reciprocal() * 127.0`, each step rounded to the tensor's type.
template <int MODE>
__device__ __forceinline__ float act_scale_from_absmax(float absmax, float eps) {
    float mx = rnd<MODE>(fmaxf(absmax, eps));
    float r = rnd<MODE>(__frcp_rn(mx));
    return rnd<MODE>(__fmul_rn(r, 127.0f));
}

template <int MODE>
__device__ __forceinline__ int quantize_one(float x, float s) {
    float v = rnd<MODE>(__fmul_rn(x, s));
    int q = __float2int_rn(v);  // round half to even
    return max(-128, min(127, q));
}

// ---- loads of 8 consecutive elements as fp32 ----
template <int DT>
struct Elem;
template <>
struct Elem<WF_F32> {
    using type = float;
    static constexpr int VEC = 4;  // elements per 16-byte load
};
template <>
struct Elem<WF_F16> {
    using type = __half;
    static constexpr int VEC = 8;
};
template <>
struct Elem<WF_BF16> {
    using type = __nv_bfloat16;
    static constexpr int VEC = 8;
};

// Loads 8 consecutive elements starting at p (16-byte aligned for 2-byte types,
// 32-byte aligned pairs of loads for fp32) into f[8].
template <int DT>
__device__ __forceinline__ void load8(const void* base, int64_t elem_off, float (&f)[8]) {
    if constexpr (DT == WF_F32) {
        const float4* p = reinterpret_cast<const float4*>(static_cast<const float*>(base) + elem_off);
        float4 a = __ldg(p), b = __ldg(p + 1);
        f[0] = a.x; f[1] = a.y; f[2] = a.z; f[3] = a.w;
        f[4] = b.x; f[5] = b.y; f[6] = b.z; f[7] = b.w;
    } else if constexpr (DT == WF_BF16) {
        uint4 u = __ldg(reinterpret_cast<const uint4*>(static_cast<const __nv_bfloat16*>(base) + elem_off));
        const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            f[2 * i] = __uint_as_float(w[i] << 16);
            f[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
        }
    } else {
        uint4 u = __ldg(reinterpret_cast<const uint4*>(static_cast<const __half*>(base) + elem_off));
        const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            __half2 h = *reinterpret_cast<const __half2*>(&w[i]);
            float2 v = __half22float2(h);
            f[2 * i] = v.x;
            f[2 * i + 1] = v.y;
        }
    }
}

template <int DT>
__device__ __forceinline__ float load1(const void* base, int64_t off) {
    if constexpr (DT == WF_F32) return static_cast<const float*>(base)[off];
    if constexpr (DT == WF_BF16) return __bfloat162float(static_cast<const __nv_bfloat16*>(base)[off]);
    return __half2float(static_cast<const __half*>(base)[off]);
}

__device__ __forceinline__ float load1_rt(const void* base, int dt, int64_t off) {
    if (dt == WF_F32) return static_cast<const float*>(base)[off];
    if (dt == WF_BF16) return __bfloat162float(static_cast<const __nv_bfloat16*>(base)[off]);
    return __half2float(static_cast<const __half*>(base)[off]);
}

__device__ __forceinline__ void store1_rt(void* base, int dt, int64_t off, float v) {
    if (dt == WF_F32)
        static_cast<float*>(base)[off] = v;
    else if (dt == WF_BF16)
        static_cast<__nv_bfloat16*>(base)[off] = __float2bfloat16_rn(v);
    else
        static_cast<__half*>(base)[off] = __float2half_rn(v);
}

// The rescale of the integer accumulator; the order of the fp32 operations is
// part of the contract: (float(acc) * inv_sx) * s_w, then + bias.
__device__ __forceinline__ float rescale(int acc, float inv_sx, float s_w) {
    return __fmul_rn(__fmul_rn(static_cast<float>(acc), inv_sx), s_w);
}

}  // namespace wf
