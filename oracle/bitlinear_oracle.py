"""CPU oracle for the ternary BitLinear hot path (numpy restatement).

TEST INFRASTRUCTURE ONLY.  This module restates, in plain numpy, the arithmetic
of the reference's BitLinear path so that the CUDA kernels can be checked
bit-for-bit on a machine where the reference sources are absent.  Nothing in the
shipped package imports it; only the tests, the smoke check and the CPU-baseline
leg of the benchmark do.

Parity status: PINNED.  `tests/golden/make_golden.py` runs the reference's own
functions (PyTorch ``BitLinear``, ``ternary_weight_quantization_no_scale``, the
packers of the inference package and the compiled ``bitnet_gemv.cpp``) on seeded
inputs and stores their outputs; `tests/test_oracle_golden.py` checks every
function below against those outputs.

Reference files restated here (paths inside the reference project):
  packages/training/src/wrinklefree/models/bitlinear.py
  packages/training/src/wrinklefree/quantization/weight_quant.py
  packages/training/src/wrinklefree/quantization/activation_quant.py
  packages/inference/extern/sglang-bitnet/sgl-kernel/csrc/bitnet/bitnet_gemv.cpp
  packages/inference/extern/sglang-bitnet/sgl-kernel/python/sgl_kernel/quantization/bitnet.py
  packages/inference/scripts/convert_to_sglkernel.py
  packages/inference/src/wrinklefree_inference/kernels/native.py
  packages/inference/src/wrinklefree_inference/sglang_backend/bitnet_quantization.py
  packages/inference/tests/test_bitnet_core.py
"""
from __future__ import annotations

import numpy as np

EPS = np.float32(1e-5)  # bitlinear.py:41 (module default eps)

# --------------------------------------------------------------------------
# reduced-precision helpers (numpy has no bfloat16)
# --------------------------------------------------------------------------


def bf16_round(x: np.ndarray) -> np.ndarray:
    """Round fp32 values to the nearest bfloat16 (ties to even), returned as fp32."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    u = x.view(np.uint32).astype(np.uint64)
    lsb = (u >> 16) & 1
    r = ((u + 0x7FFF + lsb) >> 16) << 16
    out = r.astype(np.uint32).view(np.float32).copy()
    nan = np.isnan(x)
    if nan.any():
        out[nan] = np.float32(np.nan)
    return out.reshape(x.shape)


def fp16_round(x: np.ndarray) -> np.ndarray:
    """Round fp32 values to the nearest IEEE half (ties to even), returned as fp32."""
    with np.errstate(over="ignore"):
        return np.asarray(x, dtype=np.float32).astype(np.float16).astype(np.float32)


def _rounder(dtype: str):
    if dtype == "f32":
        return lambda v: np.asarray(v, dtype=np.float32)
    if dtype == "bf16":
        return bf16_round
    if dtype == "f16":
        return fp16_round
    raise ValueError(f"unknown dtype {dtype!r}")


# --------------------------------------------------------------------------
# a1: weight ternarization
# --------------------------------------------------------------------------


def absmean_scale(w: np.ndarray, eps: float = 1e-5) -> np.float32:
    """Per-tensor absmean, clamped below by eps (weight_quant.py:52, :59-70).

    The sum is carried in fp64 and rounded once to fp32, which is the correctly
    rounded mean.  torch's fp32 ``mean`` may sit one ulp away (its summation
    order is an implementation detail); the golden test records that distance.
    """
    w = np.asarray(w, dtype=np.float32)
    m = np.float32(np.abs(w.astype(np.float64)).sum() / w.size) if w.size else np.float32(0)
    return np.float32(max(m, np.float32(eps)))


def ternarize_with_scale(w: np.ndarray, scale: np.float32) -> np.ndarray:
    """codes = clamp(round_half_even(w / scale), -1, 1) in fp32 (weight_quant.py:53-54)."""
    w = np.asarray(w, dtype=np.float32)
    q = np.rint(w / np.float32(scale))
    return np.clip(q, -1, 1).astype(np.int8)


def ternarize_absmean(w: np.ndarray, eps: float = 1e-5):
    """fp32 ternarization: returns (codes int8 in {-1,0,1}, absmean fp32).

    Follows ``ternary_weight_quantization_no_scale`` (weight_quant.py:35-56).
    """
    s = absmean_scale(w, eps)
    return ternarize_with_scale(w, s), s


def ternarize_cast_first(w: np.ndarray, dtype: str = "bf16", eps: float = 1e-5):
    """Ternarization as ``BitLinear.forward`` performs it for a low-precision input.

    bitlinear.py:103 casts the latent weight to x.dtype first, then :59-62
    compute ``scale = 1/clamp(mean|w|, eps)`` and ``round(w*scale)`` with every
    intermediate rounded to that dtype.  Returns (codes, dequant) where dequant
    is the value ``1/scale`` as the reference materialises it (``±1/scale`` are
    the non-zero entries of ``w_quant``), as fp32.
    """
    rnd = _rounder(dtype)
    wl = rnd(w)
    mean = rnd(np.float32(np.abs(wl.astype(np.float64)).sum() / wl.size))
    mean = rnd(np.maximum(mean, np.float32(eps)))
    scale = rnd(np.float32(1.0) / mean)
    q = np.clip(np.rint(rnd(wl * scale)), -1, 1)
    dequant = rnd(np.float32(1.0) / scale)
    return q.astype(np.int8), np.float32(dequant), np.float32(scale)


# --------------------------------------------------------------------------
# a2: activation quantization
# --------------------------------------------------------------------------


def act_quant_per_token(x: np.ndarray, dtype: str = "f32", eps: float = 1e-5):
    """Per-token absmax int8 quantization (bitlinear.py:79-82).

    ``x`` holds values already representable in ``dtype`` (given as fp32).
    Every intermediate is rounded to ``dtype`` exactly where torch would round.
    ``127.0 / t`` on a tensor is evaluated by torch as ``t.reciprocal() * 127.0``
    (two roundings), so ``scale = rnd(rnd(1/clamp(absmax, eps)) * 127)``; then
    ``rnd(x*scale)``, round-half-even and clamp to [-128, 127].  Returns (q int8 [M,K], scale fp32 [M]) where scale is
    the rounded quantization multiplier (the reference divides by it again to
    dequantize).
    """
    rnd = _rounder(dtype)
    x = np.asarray(x, dtype=np.float32)
    x2 = x.reshape(-1, x.shape[-1])
    absmax = np.abs(x2).max(axis=1)
    absmax = rnd(np.maximum(absmax, np.float32(eps)))
    scale = rnd(rnd(np.float32(1.0) / absmax) * np.float32(127.0))
    q = np.clip(np.rint(rnd(x2 * scale[:, None])), -128, 127).astype(np.int8)
    return q.reshape(x.shape), scale.astype(np.float32)


def act_quant_per_tensor(x: np.ndarray):
    """Per-tensor absmax quantization of the sgl-kernel CPU path.

    bitnet_gemv.cpp:880-913 (AVX-512 branch): ``max<1e-6 => 1``,
    ``scale = max/127`` is returned, values are multiplied by ``127/max`` and
    converted with round-to-nearest-even and int8 saturation.
    Returns (q int8 same shape, scale fp32 scalar).
    """
    x = np.asarray(x, dtype=np.float32)
    mx = np.float32(np.abs(x).max()) if x.size else np.float32(0)
    if mx < np.float32(1e-6):
        mx = np.float32(1.0)
    scale = np.float32(mx / np.float32(127.0))
    inv = np.float32(np.float32(127.0) / mx)
    q = np.clip(np.rint(x * inv), -128, 127).astype(np.int8)
    return q, scale


# --------------------------------------------------------------------------
# a3/a5/a6: integer contraction and rescale
# --------------------------------------------------------------------------


def int_gemm(q: np.ndarray, codes: np.ndarray) -> np.ndarray:
    """acc[m,n] = sum_k q[m,k]*codes[n,k], exact, int32."""
    q2 = q.reshape(-1, q.shape[-1]).astype(np.int32)
    return (q2 @ codes.astype(np.int32).T).astype(np.int32)


def rescale(acc: np.ndarray, act_scale: np.ndarray, w_scale, bias=None) -> np.ndarray:
    """y = (float(acc) * (1/act_scale[m])) * w_scale (+ bias), all fp32.

    The order is fixed: integer -> fp32, times the reciprocal of the per-token
    quantization multiplier, times the weight scale, then the bias.
    """
    inv = (np.float32(1.0) / np.asarray(act_scale, dtype=np.float32)).astype(np.float32)
    y = (acc.astype(np.float32) * inv[:, None]).astype(np.float32) * np.float32(w_scale)
    if bias is not None:
        y = y + np.asarray(bias, dtype=np.float32)[None, :]
    return y.astype(np.float32)


def bitlinear_forward(x, w, dtype="f32", bias=None, eps=1e-5, weight_mode="f32"):
    """Whole path on integers: returns dict(codes, w_scale, q, act_scale, acc, y).

    weight_mode "f32": codes and scale of ``ternary_weight_quantization_no_scale``.
    weight_mode "cast_first": codes and dequantization value as ``BitLinear.forward``
    forms them when its input has the low-precision ``dtype`` (bitlinear.py:103-107);
    a few codes per thousand differ between the two, so the low-precision reference
    forward is matched to 1e-2 only in this mode.
    """
    if weight_mode == "cast_first" and dtype != "f32":
        codes, s_w, _ = ternarize_cast_first(w, dtype, eps)
    else:
        codes, s_w = ternarize_absmean(w, eps)
    q, s_x = act_quant_per_token(x, dtype, eps)
    acc = int_gemm(q, codes)
    y = rescale(acc, s_x.reshape(-1), s_w, bias)
    return dict(codes=codes, w_scale=s_w, q=q, act_scale=s_x, acc=acc, y=y)


def bitlinear_forward_float(x, w, dtype="f32", bias=None, eps=1e-5):
    """Literal fake-quant forward of bitlinear.py:99-113 at lambda=1 in ``dtype``.

    The GEMM itself is carried in fp64 and rounded once to ``dtype`` (the
    reference's summation order inside F.linear is library-defined).
    """
    rnd = _rounder(dtype)
    x = rnd(x)
    x2 = x.reshape(-1, x.shape[-1])
    if dtype == "f32":
        wl = np.asarray(w, dtype=np.float32)
        mean = np.float32(max(np.float32(np.abs(wl.astype(np.float64)).sum() / wl.size), np.float32(eps)))
        scale = np.float32(1.0) / mean
        wq = (np.clip(np.rint(wl * scale), -1, 1) / scale).astype(np.float32)
    else:
        codes, dq, _ = ternarize_cast_first(w, dtype, eps)
        wq = codes.astype(np.float32) * dq
    q, s = act_quant_per_token(x2, dtype, eps)
    xq = rnd(q.astype(np.float32) / s[:, None])
    y = xq.astype(np.float64) @ wq.astype(np.float64).T
    if bias is not None:
        y = y + rnd(bias).astype(np.float64)[None, :]
    return rnd(y.astype(np.float32))


# --------------------------------------------------------------------------
# packed layouts (code = w + 1 in {0,1,2} everywhere)
# --------------------------------------------------------------------------


def pack_wf16(codes: np.ndarray) -> np.ndarray:
    """The GPU layout of this library: row-major [N, K/4] bytes, K % 16 == 0.

    Each little-endian 32-bit word holds 16 consecutive weights k0..k0+15:
    byte b (0..3), bit pair j (bits 2j+1:2j) holds weight k0 + 4*j + b.
    ``(word >> 2j) & 0x03030303`` therefore yields weights k0+4j .. k0+4j+3 as
    four bytes in memory order, ready for a 4-way int8 dot product.
    """
    n, k = codes.shape
    assert k % 16 == 0
    c = (codes.astype(np.int16) + 1).astype(np.uint8).reshape(n, k // 16, 4, 4)  # [n, word, j, b]
    out = np.zeros((n, k // 16, 4), dtype=np.uint8)  # [n, word, b]
    for j in range(4):
        out |= c[:, :, j, :] << (2 * j)
    return out.reshape(n, k // 4)


def unpack_wf16(packed: np.ndarray) -> np.ndarray:
    n, kb = packed.shape
    p = packed.reshape(n, kb // 4, 4)
    c = np.zeros((n, kb // 4, 4, 4), dtype=np.int8)
    for j in range(4):
        c[:, :, j, :] = ((p >> (2 * j)) & 3).astype(np.int8) - 1
    return c.reshape(n, kb * 4)


def pack_i2s(codes: np.ndarray) -> np.ndarray:
    """I2_S block layout (convert_to_sglkernel.py:96-111; test_bitnet_core.py:56-104).

    Per 128 weights, 32 bytes: byte j bits 7:6 -> k=j, 5:4 -> j+32, 3:2 -> j+64,
    1:0 -> j+96.
    """
    n, k = codes.shape
    assert k % 128 == 0
    c = (codes.astype(np.int16) + 1).astype(np.uint8).reshape(n, k // 128, 4, 32)
    out = (c[:, :, 0, :] << 6) | (c[:, :, 1, :] << 4) | (c[:, :, 2, :] << 2) | c[:, :, 3, :]
    return out.reshape(n, k // 4).astype(np.uint8)


def unpack_i2s(packed: np.ndarray) -> np.ndarray:
    n, kb = packed.shape
    p = packed.reshape(n, kb // 32, 32)
    c = np.zeros((n, kb // 32, 4, 32), dtype=np.int8)
    for g in range(4):
        c[:, :, g, :] = ((p >> (6 - 2 * g)) & 3).astype(np.int8) - 1
    return c.reshape(n, kb * 4)


def pack_seq_lsb(codes: np.ndarray) -> np.ndarray:
    """Sequential, LSB first: byte j = k 4j..4j+3 at shifts 0,2,4,6 (native.py:181-198)."""
    n, k = codes.shape
    c = (codes.astype(np.int16) + 1).astype(np.uint8).reshape(n, k // 4, 4)
    return (c[:, :, 0] | (c[:, :, 1] << 2) | (c[:, :, 2] << 4) | (c[:, :, 3] << 6)).astype(np.uint8)


def unpack_seq_lsb(packed: np.ndarray) -> np.ndarray:
    n, kb = packed.shape
    c = np.stack([((packed >> (2 * i)) & 3) for i in range(4)], axis=-1)
    return (c.astype(np.int8) - 1).reshape(n, kb * 4)


def pack_seq_msb(codes: np.ndarray) -> np.ndarray:
    """Sequential, MSB first: byte j = k 4j..4j+3 at shifts 6,4,2,0 (bitnet_quantization.py:96-107)."""
    n, k = codes.shape
    c = (codes.astype(np.int16) + 1).astype(np.uint8).reshape(n, k // 4, 4)
    return ((c[:, :, 0] << 6) | (c[:, :, 1] << 4) | (c[:, :, 2] << 2) | c[:, :, 3]).astype(np.uint8)


def unpack_seq_msb(packed: np.ndarray) -> np.ndarray:
    n, kb = packed.shape
    c = np.stack([((packed >> (6 - 2 * i)) & 3) for i in range(4)], axis=-1)
    return (c.astype(np.int8) - 1).reshape(n, kb * 4)


def pack_hf(codes: np.ndarray) -> np.ndarray:
    """HF checkpoint layout [N/4, K]: byte (r,c) holds rows r, r+N/4, r+2N/4, r+3N/4
    at shifts 0,2,4,6 (test_bitnet_core.py:21-53)."""
    n, k = codes.shape
    assert n % 4 == 0
    c = (codes.astype(np.int16) + 1).astype(np.uint8).reshape(4, n // 4, k)
    return (c[0] | (c[1] << 2) | (c[2] << 4) | (c[3] << 6)).astype(np.uint8)


def unpack_hf(packed: np.ndarray) -> np.ndarray:
    r, k = packed.shape
    c = np.concatenate([((packed >> (2 * i)) & 3) for i in range(4)], axis=0)
    return c.astype(np.int8) - 1


# --------------------------------------------------------------------------
# a5-a7: the sgl-kernel operator semantics on I2_S weights
# --------------------------------------------------------------------------


def vec_dot_i2_i8(packed_row_i2s: np.ndarray, act: np.ndarray) -> np.float32:
    """bitnet_vec_dot_i2_i8 (bitnet_gemv.cpp:325-808): sum(code*a) - sum(a), as float."""
    codes_u = unpack_i2s(packed_row_i2s.reshape(1, -1)).astype(np.int32) + 1
    a = act.astype(np.int32)
    return np.float32(int((codes_u[0] * a).sum() - a.sum()))


def bitnet_gemm_i2s(packed_i2s: np.ndarray, act: np.ndarray, scale: float) -> np.ndarray:
    """bitnet_gemm semantics after the Python transpose fix
    (sgl_kernel/quantization/bitnet.py:114-152): [batch, out] fp32 = acc * scale."""
    t = unpack_i2s(packed_i2s).astype(np.int32)
    acc = act.reshape(-1, act.shape[-1]).astype(np.int32) @ t.T
    return (acc.astype(np.float32) * np.float32(scale)).astype(np.float32)
