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


def reference_root():
    """A checkout of the reference project: $WF_REFERENCE_ROOT, else a directory named `reference` beside the
    repository; None when neither holds the kernel sources."""
    probe = os.path.join("packages", "inference", "extern", "sglang-bitnet", "sgl-kernel", "csrc", "bitnet", "bitnet_gemv.cpp")
    for cand in (os.environ.get("WF_REFERENCE_ROOT"), os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference")):
        if cand and os.path.exists(os.path.join(cand, probe)):
            return cand
    return None


def _system_compiler(name: str) -> str:
    """The distribution's compiler when present (it carries OpenMP), else whatever PATH offers."""
    sys_path = os.path.join(os.sep, "usr", "bin", name)
    return sys_path if os.path.exists(sys_path) else name


def build(quiet: bool = True) -> None:
    """Compile the C oracle and, when a reference checkout is found, oracle/_ref."""
    env = dict(os.environ, CC=_system_compiler("gcc"), CXX=_system_compiler("g++"))
    cmd = ["make", "-C", HERE]
    ref = reference_root()
    if ref:
        cmd.append(f"REF={ref}")
    r = subprocess.run(cmd, env=env, capture_output=True, text=True)
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

    def set_num_threads(self, n: int) -> None:
        self.lib.ref_set_num_threads(_i32(n))

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


class GgmlReference:
    """BitNet.cpp's I2_S routines (ggml-bitnet-mad.cpp compiled behind ggml_shim.cpp)."""

    def __init__(self, lib):
        self.lib = lib
        lib.ggml_ref_num_threads.restype = _i32
        lib.ggml_ref_quantize_i2_s.restype = C.c_size_t
        lib.ggml_ref_quantize_i2_s.argtypes = [_p, _p, _i64, _i64]
        lib.ggml_ref_vec_dot.restype = _f32
        lib.ggml_ref_vec_dot.argtypes = [_i32, _p, _p]
        lib.ggml_ref_mul_mat.argtypes = [_i32, _i32, _i32, _p, _p, _p, _p, _p, _f32]

    def num_threads(self) -> int:
        return int(self.lib.ggml_ref_num_threads())

    def set_num_threads(self, n: int) -> None:
        self.lib.ggml_ref_set_num_threads(_i32(n))

    def quantize_i2_s(self, w):
        """Returns (packed uint8 [N, K/4] in the I2_S block order, scale)."""
        w = np.ascontiguousarray(w, dtype=np.float32)
        n, k = w.shape
        buf = np.zeros(n * k // 4 + 64, dtype=np.uint8)
        self.lib.ggml_ref_quantize_i2_s(_ptr(w), _ptr(buf), _i64(n), _i64(k))
        scale = buf[n * k // 4:n * k // 4 + 4].view(np.float32)[0]
        return buf[:n * k // 4].reshape(n, k // 4).copy(), np.float32(scale)

    def vec_dot(self, packed_row, act):
        packed_row = np.ascontiguousarray(packed_row, dtype=np.uint8)
        act = np.ascontiguousarray(act, dtype=np.int8)
        return np.float32(self.lib.ggml_ref_vec_dot(_i32(act.size), _ptr(packed_row), _ptr(act)))

    def mul_mat(self, packed, act, act_sums, act_scales, w_scale):
        """[batch, rows] fp32 = (dot - act_sum) / act_scale * w_scale, rows in an OpenMP loop."""
        packed = np.ascontiguousarray(packed, dtype=np.uint8)
        act = np.ascontiguousarray(act, dtype=np.int8)
        act_sums = np.ascontiguousarray(act_sums, dtype=np.float32)
        act_scales = np.ascontiguousarray(act_scales, dtype=np.float32)
        rows, kb = packed.shape
        b = act.shape[0]
        out = np.empty((b, rows), dtype=np.float32)
        self.lib.ggml_ref_mul_mat(_i32(rows), _i32(kb * 4), _i32(b), _ptr(out), _ptr(packed), _ptr(act), _ptr(act_sums),
                                  _ptr(act_scales), _f32(w_scale))
        return out


def load_ggml_reference():
    path = os.path.join(HERE, "_ref", "libref_ggml_mad_avx2.so")
    if "avx2" in _cpu_flags() and os.path.exists(path):
        return GgmlReference(C.CDLL(path))
    return None
