"""ctypes binding of libwf_b200.so (the C ABI declared in include/wf_b200.h).

There is no fallback: if the library has not been built, or a call fails, a
RuntimeError is raised with the library's own message.
"""
from __future__ import annotations

import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libwf_b200.so")

# constants of include/wf_b200.h
WF_F32, WF_F16, WF_BF16, WF_I8 = 0, 1, 2, 3
LAYOUT_WF16, LAYOUT_I2S, LAYOUT_SEQ_LSB, LAYOUT_SEQ_MSB, LAYOUT_HF = 0, 1, 2, 3, 4
PACK_FP32, PACK_CAST_BF16, PACK_CAST_F16 = 0, 1, 2
ACT_PER_TOKEN, ACT_PER_TENSOR = 0, 1
MAXABS_HALF, MAXABS_SIGN = 0, 1
X_PLAIN, X_SILU, X_RELU2, X_NORM = 0, 1, 2, 3
FLAG_PDL = 1
FLAG_X_READY = 2
FLAG_PREFILL_PAIR, FLAG_PREFILL_SINGLE = 4, 8
FLAG_WS_READY = 16

_i64, _int, _f32, _p, _sz, _u32 = C.c_int64, C.c_int, C.c_float, C.c_void_p, C.c_size_t, C.c_uint



class Problem(C.Structure):
    """Mirror of `wf_problem` (include/wf_b200.h)."""

    _fields_ = [("x", _p), ("x_scale", _p), ("codes", _p), ("w_scale", _p), ("bias", _p), ("y", _p), ("acc_out", _p),
                ("ldx", _i64), ("ldy", _i64), ("M", C.c_int32), ("N", C.c_int32), ("K", C.c_int32),
                ("x_dtype", C.c_int32), ("y_dtype", C.c_int32), ("bias_dtype", C.c_int32), ("layout", C.c_int32),
                ("w_scale_host", _f32), ("eps", _f32),
                ("_item_begin", C.c_int32), ("_row_items", C.c_int32), ("_chunks", C.c_int32), ("_kb_full", C.c_int32),
                ("_tail_bytes", C.c_int32), ("_kb_seg", C.c_int32), ("_ksegs", C.c_int32),
                ("x2", _p), ("norm_w", _p), ("h_out", _p), ("x_mode", C.c_int32), ("norm_eps", _f32), ("prefetch", _p), ("prefetch_bytes", _i64), ("xchg", _p),
                ("_tmap_main", C.c_uint64 * 16), ("_tmap_last", C.c_uint64 * 16), ("_tmap_tail", C.c_uint64 * 16)]


assert C.sizeof(Problem) == 576


def aligned_problem_array(n: int):
    """A ctypes array of n Problem structs starting on a 64-byte boundary (returns array, keep-alive buffer)."""
    raw = (C.c_char * (n * C.sizeof(Problem) + 64))()
    addr = (C.addressof(raw) + 63) // 64 * 64
    return (Problem * n).from_address(addr), raw


_SIGNATURES = {
    "wf_version": (_int, []),
    "wf_last_error": (C.c_char_p, []),
    "wf_device_check": (_int, []),
    "wf_probe_i8_mma": (_int, [_int, _int, C.POINTER(C.c_double), C.POINTER(C.c_double)]),
    "wf_pack_scratch_bytes": (_sz, [_i64, _i64]),
    "wf_pack_ternary": (_int, [_p, _int, _i64, _i64, _i64, _int, _f32, _p, _p, _p, _sz, _p]),
    "wf_pack_noalloc_scratch_bytes": (_sz, []),
    "wf_pack_ternary_noalloc": (_int, [_p, _int, _i64, _i64, _i64, _int, _f32, _p, _p, _p]),
    "wf_repack": (_int, [_p, _int, _p, _int, _i64, _i64, _p]),
    "wf_quantize_maxabs": (_int, [_p, _int, _i64, _i64, _i64, _int, _int, _p, _p, _p]),
    "wf_pack_codes": (_int, [_p, _p, _int, _i64, _i64, _p]),
    "wf_unpack_codes": (_int, [_p, _int, _p, _i64, _i64, _p]),
    "wf_act_quant_i8": (_int, [_p, _int, _i64, _i64, _i64, _int, _f32, _p, _p, _p, _p]),
    "wf_bitlinear_decode": (_int, [_p, _int, _i64, _p, _p, _int, _p, _f32, _p, _int, _p, _int, _i64, _p, _i64, _i64, _i64,
                                   _f32, _u32, _p]),
    "wf_bitlinear_decode_plan": (_int, [_p, _int]),
    "wf_bitlinear_decode_grouped": (_int, [_p, _p, _int, _u32, _p]),
    "wf_device_status": (_int, []),
    "wf_prefill_workspace_bytes": (_sz, [_i64, _i64]),
    "wf_bitlinear_prefill": (_int, [_p, _int, _i64, _p, _p, _int, _p, _f32, _p, _int, _p, _int, _i64, _p, _i64, _i64, _i64,
                                    _f32, _p, _sz, _u32, _p]),
    "wf_add_rmsnorm_bf16": (_int, [_p, _p, _p, _p, _i64, _i64, _f32, _u32, _p]),
    "wf_rope_kv_bf16": (_int, [_p, _p, _p, _p, _p, _p, _p, _p, _i64, _int, _int, _int, _int, _u32, _p]),
    "wf_act_mul_bf16": (_int, [_p, _p, _p, _i64, _int, _u32, _p]),
    "wf_attn_decode_workspace_bytes": (_sz, [_i64, _int, _int, _int, _int]),
    "wf_attn_decode_bf16": (_int, [_p, _p, _p, _p, _p, _i64, _int, _int, _int, _int, _f32, _p, _sz, _u32, _p]),
    "wf_add_rmsnorm_quant_bf16": (_int, [_p, _p, _p, _p, _p, _p, _i64, _i64, _f32, _f32, _u32, _p]),
    "wf_act_mul_quant_bf16": (_int, [_p, _p, _p, _p, _p, _i64, _i64, _int, _f32, _u32, _p]),
    "wf_linear_bf16": (_int, [_p, _i64, _p, _i64, _p, _int, _i64, _i64, _i64, _i64, _u32, _p]),
    "wf_ar_handle_bytes": (_int, []),
    "wf_ar_init": (_int, [_int, _int, _sz, C.POINTER(C.c_void_p), _p]),
    "wf_ar_connect": (_int, [_p, _p]),
    "wf_ar_allreduce": (_int, [_p, _p, _p, _i64, _int, _u32, _p]),
    "wf_ar_status": (_int, [_p, C.POINTER(C.c_int)]),
    "wf_ar_xchg": (_int, [_p, C.POINTER(C.c_void_p)]),
    "wf_ar_reduce_add_rmsnorm": (_int, [_p, _p, _p, _p, _i64, _i64, _f32, _u32, _p]),
    "wf_ar_reduce_add_rmsnorm_quant": (_int, [_p, _p, _p, _p, _p, _p, _i64, _i64, _f32, _f32, _u32, _p]),
    "wf_ar_step": (_int, [_p, C.POINTER(C.c_uint)]),
    "wf_ar_set_step": (_int, [_p, _u32]),
    "wf_ar_destroy": (_int, [_p]),
    "wf_bitlinear_prefill_batched": (_int, [_p, _int, _i64, _p, _int, _p, _i64, _p, _int, _i64, _p, _i64, _i64, _i64, _i64, _f32,
                                            _p, _sz, _u32, _p]),
    "wf_prefill_quantize": (_int, [_p, _int, _i64, _i64, _i64, _f32, _p, _sz, _u32, _p]),
}

_lib = None


def exported_symbols():
    """Names every build of the library must export (checked by the CPU tests)."""
    return sorted(_SIGNATURES)


def lib():
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                f"{LIB_PATH} is missing: build it with `python __graft_entry__.py build` "
                "(there is no CPU or PyTorch fallback for these operators)"
            )
        handle = C.CDLL(LIB_PATH)
        for name, (res, args) in _SIGNATURES.items():
            fn = getattr(handle, name)
            fn.restype = res
            fn.argtypes = args
        _lib = handle
    return _lib


def check(rc: int, what: str) -> None:
    if rc != 0:
        msg = lib().wf_last_error().decode("utf-8", "replace")
        raise RuntimeError(f"{what} failed (code {rc}): {msg}")
