"""ctypes loaders for the C oracle and for the reference's own CPU kernel.

TEST INFRASTRUCTURE ONLY (see bitlinear_oracle.py).  ``load_oracle()`` returns
the plain-C restatement (oracle/wf_oracle.c); ``load_reference()`` returns the
reference's ``bitnet_gemv.cpp`` compiled behind ``ref_shim.cpp`` or None when
no prebuilt copy exists.  ``build()`` runs the Makefile.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
_i64, _i32, _f32 = C.c_int64, C.c_int, C.c_float
_p = C.c_void_p


def build(quiet: bool = True) -> None:
    """Compile the C oracle and, when the reference tree is present, oracle/_ref."""
    env = dict(os.environ, CC="/usr/bin/gcc", CXX="/usr/bin/g++")
    r = subprocess.run(["make", "-C", HERE], env=env, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("oracle build failed:\n" + r.stdout + r.stderr)
    if not quiet:
        print(r.stdout)


def _ptr(a: np.ndarray):
    return a.ctypes.data_as(_p)


class Oracle:
    def __init__(self, lib):
        self.lib = lib
        lib.wfo_absmean.restype = _f32
        lib.wfo_absmean.argtypes = [_p, _i64, _f32]
        lib.wfo_num_threads.restype = _i32

    def num_threads(self) -> int:
        return int(self.lib.wfo_num_threads())

    def absmean(self, w, eps=1e-5):
        w = np.ascontiguousarray(w, dtype=np.float32)
        return np.float32(self.lib.wfo_absmean(_ptr(w), _i64(w.size), _f32(eps)))

    def ternarize(self, w, scale):
        w = np.ascontiguousarray(w, dtype=np.float32)
        out = np.empty(w.shape, dtype=np.int8)
        self.lib.wfo_ternarize(_ptr(w), _i64(w.size), _f32(scale), _ptr(out))
        return out

    def pack_wf16(self, codes):
        codes = np.ascontiguousarray(codes, dtype=np.int8)
        n, k = codes.shape
        out = np.empty((n, k // 4), dtype=np.uint8)
        self.lib.wfo_pack_wf16(_ptr(codes), _i64(n), _i64(k), _ptr(out))
        return out

    def pack_i2s(self, codes):
        codes = np.ascontiguousarray(codes, dtype=np.int8)
        n, k = codes.shape
        out = np.empty((n, k // 4), dtype=np.uint8)
        self.lib.wfo_pack_i2s(_ptr(codes), _i64(n), _i64(k), _ptr(out))
        return out

    def act_quant(self, x, mode=0, eps=1e-5):
        x = np.ascontiguousarray(x, dtype=np.float32)
        m, k = x.shape
        q = np.empty((m, k), dtype=np.int8)
        s = np.empty((m,), dtype=np.float32)
        self.lib.wfo_act_quant(_ptr(x), _i64(m), _i64(k), _i32(mode), _f32(eps), _ptr(q), _ptr(s))
        return q, s

    def int_gemm(self, q, codes):
        q = np.ascontiguousarray(q, dtype=np.int8)
        codes = np.ascontiguousarray(codes, dtype=np.int8)
        m, k = q.shape
        n = codes.shape[0]
        acc = np.empty((m, n), dtype=np.int32)
        self.lib.wfo_int_gemm(_ptr(q), _ptr(codes), _i64(m), _i64(n), _i64(k), _ptr(acc))
        return acc

    def gemm_wf16(self, q, packed):
        q = np.ascontiguousarray(q, dtype=np.int8)
        packed = np.ascontiguousarray(packed, dtype=np.uint8)
        m, k = q.shape
        n = packed.shape[0]
        acc = np.empty((m, n), dtype=np.int32)
        self.lib.wfo_gemm_wf16(_ptr(q), _ptr(packed), _i64(m), _i64(n), _i64(k), _ptr(acc))
        return acc

    def rescale(self, acc, act_scale, w_scale, bias=None):
        acc = np.ascontiguousarray(acc, dtype=np.int32)
        act_scale = np.ascontiguousarray(act_scale, dtype=np.float32)
        m, n = acc.shape
        y = np.empty((m, n), dtype=np.float32)
        b = np.ascontiguousarray(bias, dtype=np.float32) if bias is not None else None
        self.lib.wfo_rescale(_ptr(acc), _ptr(act_scale), _f32(w_scale), _ptr(b) if b is not None else None,
                             _i64(m), _i64(n), _ptr(y))
        return y


class Reference:
    """The reference's own bitnet_gemv.cpp (I2_S weights, K % 128 == 0)."""

    def __init__(self, lib, flavour):
        self.lib = lib
        self.flavour = flavour
        lib.ref_num_threads.restype = _i32

    def num_threads(self) -> int:
        return int(self.lib.ref_num_threads())

    def vec_dot(self, packed_row, act):
        packed_row = np.ascontiguousarray(packed_row, dtype=np.uint8)
        act = np.ascontiguousarray(act, dtype=np.int8)
        r = C.c_float(0)
        rc = self.lib.ref_vec_dot_i2_i8(_i32(act.size), C.byref(r), _ptr(packed_row), _ptr(act))
        if rc:
            raise ValueError("reference kernel rejected the shape")
        return np.float32(r.value)

    def gemm(self, packed, act, scale):
        """Returns [batch, out] fp32 (the kernel writes [out, batch]; transposed here as
        sgl_kernel/quantization/bitnet.py:139-145 does)."""
        packed = np.ascontiguousarray(packed, dtype=np.uint8)
        act = np.ascontiguousarray(act, dtype=np.int8)
        n_out, kb = packed.shape
        b, k = act.shape
        out = np.empty((n_out, b), dtype=np.float32)
        rc = self.lib.ref_gemm_i2_i8(_i32(n_out), _i32(b), _i32(k), _ptr(out), _ptr(packed), _ptr(act), _f32(scale))
        if rc:
            raise ValueError("reference kernel rejected the shape")
        return np.ascontiguousarray(out.T)

    def gemv(self, packed, act, scale):
        packed = np.ascontiguousarray(packed, dtype=np.uint8)
        act = np.ascontiguousarray(act, dtype=np.int8)
        n_out, kb = packed.shape
        out = np.empty((n_out,), dtype=np.float32)
        rc = self.lib.ref_gemv_rows(_i32(n_out), _i32(kb * 4), _ptr(out), _ptr(packed), _ptr(act), _f32(scale))
        if rc:
            raise ValueError("reference kernel rejected the shape")
        return out

    def quantize_activations(self, x):
        x = np.ascontiguousarray(x, dtype=np.float32)
        q = np.empty(x.shape, dtype=np.int8)
        s = C.c_float(0)
        self.lib.ref_quantize_activations_i8(_i32(x.size), _ptr(q), _ptr(x), C.byref(s))
        return q, np.float32(s.value)


def load_oracle() -> Oracle:
    path = os.path.join(HERE, "_build", "libwf_oracle.so")
    if not os.path.exists(path):
        build()
    return Oracle(C.CDLL(path))


def _cpu_flags() -> set:
    try:
        with open("/proc/cpuinfo") as f:
            for line in f:
                if line.startswith("flags"):
                    return set(line.split(":", 1)[1].split())
    except OSError:
        pass
    return set()


def load_reference():
    flags = _cpu_flags()
    order = []
    if {"avx512f", "avx512bw", "avx512vl"} <= flags:
        order.append("avx512")
    if "avx2" in flags:
        order.append("avx2")
    for fl in order:
        path = os.path.join(HERE, "_ref", f"libref_bitnet_{fl}.so")
        if os.path.exists(path):
            return Reference(C.CDLL(path), fl)
    return None
