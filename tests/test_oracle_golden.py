"""The CPU oracle against the reference's own outputs (golden vectors) and the
known-answer tests of the reference's test-suite.  No GPU."""
import os

import numpy as np
import pytest
import torch

import inputs as gi
from oracle import bitlinear_oracle as O

GOLD = os.path.join(os.path.dirname(__file__), "golden")


def load(name):
    z = np.load(os.path.join(GOLD, f"{name}.npz"))
    x, w = gi.make_inputs(name)
    assert gi.sha(x.numpy(), w.numpy()) == str(z["input_sha"]), "seeded inputs changed; regenerate the golden files"
    return z, x, w


def ulp_dist(a, b):
    ia = np.array([a], dtype=np.float32).view(np.int32)[0]
    ib = np.array([b], dtype=np.float32).view(np.int32)[0]
    return abs(int(ia) - int(ib))


@pytest.mark.parametrize("name", list(gi.CASES))
def test_weight_codes_and_scale(name, oracle_c):
    z, x, w = load(name)
    codes, s = O.ternarize_absmean(w.numpy())
    # torch's fp32 mean may be one ulp from the correctly rounded mean
    assert ulp_dist(s, z["w_scale_torch"]) <= 1
    # codes: identical to the reference's, both with the oracle's scale and with torch's
    assert np.array_equal(O.ternarize_with_scale(w.numpy(), z["w_scale_torch"]), z["codes"])
    assert np.array_equal(codes, z["codes"])
    # C restatement agrees with numpy
    assert oracle_c.absmean(w.numpy()) == s
    assert np.array_equal(oracle_c.ternarize(w.numpy(), s), codes)
    # the forward's fp32 cast-first quantization (w*(1/s)) carries the same codes
    assert np.array_equal(z["codes_fwd_f32"], z["codes"])


@pytest.mark.parametrize("name", list(gi.CASES))
@pytest.mark.parametrize("dt", ["f32", "bf16", "f16"])
def test_activation_integers(name, dt, oracle_c):
    z, x, w = load(name)
    tdt = {"f32": torch.float32, "bf16": torch.bfloat16, "f16": torch.float16}[dt]
    xd = x.to(tdt).float().numpy()
    q, s = O.act_quant_per_token(xd, dt)
    assert np.array_equal(q, z[f"q_{dt}"])
    assert np.array_equal(s, z[f"act_scale_{dt}"])
    if dt != "f16":
        q2, s2 = oracle_c.act_quant(xd, {"f32": 0, "bf16": 1}[dt])
        assert np.array_equal(q2, q) and np.array_equal(s2, s)


def test_bf16_activation_reaches_minus_128():
    # a property of the reference in bf16 that the fp32 formula does not show
    z, _, _ = load("c1")
    assert z["q_bf16"].min() == -128 and z["q_f32"].min() >= -127


@pytest.mark.parametrize("name", list(gi.CASES))
def test_cast_first_codes(name):
    z, x, w = load(name)
    for dt in ("bf16", "f16"):
        codes, dq, _ = O.ternarize_cast_first(w.numpy(), dt)
        assert np.array_equal(codes, z[f"codes_fwd_{dt}"]), dt
        assert dq == z[f"dequant_fwd_{dt}"], dt


def norm_err(a, b):
    return float(np.abs(a - b).max() / np.abs(b).max())


@pytest.mark.parametrize("name", list(gi.CASES))
def test_forward_against_reference(name, oracle_c):
    z, x, w = load(name)
    r = O.bitlinear_forward(x.numpy(), w.numpy(), "f32")
    assert np.array_equal(r["acc"], oracle_c.int_gemm(r["q"], r["codes"]))
    assert np.array_equal(r["acc"], oracle_c.gemm_wf16(r["q"], O.pack_wf16(r["codes"])))
    # fp32 reference forward: tight
    assert norm_err(r["y"], z["y_f32"]) < 1e-5
    assert np.array_equal(oracle_c.rescale(r["acc"], r["act_scale"], r["w_scale"]), r["y"])
    rb = O.bitlinear_forward(x.numpy(), w.numpy(), "f32", bias=z["bias"])
    assert norm_err(rb["y"], z["y_bias_f32"]) < 1e-5
    # bf16 / f16 reference forward: normalised max-rel 1e-2, with the weight codes formed
    # the way the forward forms them for that dtype (cast first).  With fp32 codes a few
    # codes per thousand differ and single outputs move by several percent, so that
    # pairing is not held to an output tolerance; only the share of differing codes is.
    for dt, tdt in (("bf16", torch.bfloat16), ("f16", torch.float16)):
        xd = x.to(tdt).float().numpy()
        rr = O.bitlinear_forward(xd, w.numpy(), dt, weight_mode="cast_first")
        assert norm_err(rr["y"], z[f"y_{dt}"]) < 1e-2, dt
        yl = O.bitlinear_forward_float(xd, w.numpy(), dt)
        assert norm_err(yl, z[f"y_{dt}"]) < 1e-2, dt
        r32 = O.bitlinear_forward(xd, w.numpy(), dt)
        assert (r32["codes"] != rr["codes"]).mean() < 0.01, dt


@pytest.mark.parametrize("name", gi.I2S_CASES)
def test_i2s_cpu_kernel_semantics(name):
    """The oracle's I2_S operator semantics against the reference's compiled kernel."""
    z, x, w = load(name)
    m, k, n, _ = gi.CASES[name]
    q, s = O.act_quant_per_tensor(x.numpy())
    assert np.array_equal(q, z["i2s_q_tensor"]) and s == z["i2s_act_scale"]
    packed = O.pack_i2s(z["codes"])
    out = O.bitnet_gemm_i2s(packed, q, float(z["w_scale_torch"]))
    assert np.array_equal(out, z["i2s_gemm"])
    assert np.array_equal(out[0], z["i2s_gemv_row0"])
    assert O.vec_dot_i2_i8(packed[1], q[0]) == np.float32(O.int_gemm(q[:1], z["codes"][1:2])[0, 0])


def test_reference_kernel_live_if_present():
    """Where oracle/_ref exists, the reference kernel itself must agree with the oracle."""
    from oracle.clib import load_reference

    ref = load_reference()
    if ref is None:
        pytest.skip("oracle/_ref not built on this machine")
    rng = np.random.default_rng(5)
    codes = rng.integers(-1, 2, size=(24, 384)).astype(np.int8)
    q = rng.integers(-128, 128, size=(5, 384)).astype(np.int8)
    p = O.pack_i2s(codes)
    assert np.array_equal(ref.gemm(p, q, 0.5), O.bitnet_gemm_i2s(p, q, 0.5))
    with pytest.raises(ValueError):
        ref.vec_dot(np.zeros(16, np.uint8), np.zeros(64, np.int8))  # K % 128 != 0 is rejected


def test_packers_against_reference():
    z = np.load(os.path.join(GOLD, "packers.npz"))
    t = z["ternary"]
    w = z["w"]
    codes, s = O.ternarize_absmean(w)
    assert np.array_equal(codes, t)
    assert ulp_dist(s, z["sglkernel_scale"]) <= 1  # torch's summation order
    assert np.array_equal(O.pack_i2s(t), z["sglkernel_simd"])
    assert np.array_equal(O.pack_i2s(t), z["core_blocked"])
    assert np.array_equal(O.pack_seq_lsb(t), z["sglkernel_scalar"])
    assert np.array_equal(O.pack_seq_lsb(t), z["native_seq_lsb"])
    assert np.array_equal(O.pack_seq_lsb(t), z["patch_seq_lsb"])
    assert np.array_equal(O.pack_seq_msb(t), z["quantize_to_bitnet_msb"])
    assert np.array_equal(O.unpack_seq_msb(z["quantize_to_bitnet_msb"]).astype(np.float32), z["dequantize_bitnet"])
    assert np.array_equal(O.unpack_hf(z["hf_bytes"]), z["hf_unpacked"])
    # native.repack_hf_weights interleaves rows (i::4) instead of blocking them; pinned as a known quirk
    assert np.array_equal(O.pack_hf(O.unpack_hf(z["hf_bytes"])), z["hf_bytes"])
    for f in ("wf16", "i2s", "seq_lsb", "seq_msb", "hf"):
        assert np.array_equal(getattr(O, "unpack_" + f)(getattr(O, "pack_" + f)(t)), t)


# ---- known-answer tests restated from the reference's own test-suite ----


def test_kat_scale_is_absmean():
    # packages/training/tests/test_quantization.py:65-71
    assert O.absmean_scale(np.array([[1.0, -2.0], [3.0, -4.0]], np.float32)) == np.float32(2.5)


def test_kat_zero_weights():
    # packages/training/tests/test_quantization.py:81-87
    codes, s = O.ternarize_absmean(np.zeros((4, 16), np.float32))
    assert not codes.any() and np.isfinite(s) and s == np.float32(1e-5)


def test_kat_extreme_magnitudes():
    # packages/training/tests/test_quantization.py (1e-8 and 1e6 magnitudes), test_edge_cases.py:21-33
    rng = np.random.default_rng(1)
    for mag in (1e-8, 1e6):
        w = (rng.standard_normal((8, 64)) * mag).astype(np.float32)
        codes, s = O.ternarize_absmean(w)
        assert set(np.unique(codes)) <= {-1, 0, 1} and np.isfinite(s)
        q, sc = O.act_quant_per_token(w)
        assert np.isfinite(sc).all() and q.min() >= -128


def test_kat_per_token_independence():
    # packages/training/tests/test_paper_verification.py:112-127
    rng = np.random.default_rng(2)
    x = rng.standard_normal((4, 64)).astype(np.float32)
    q_all, s_all = O.act_quant_per_token(x)
    for i in range(4):
        qi, si = O.act_quant_per_token(x[i : i + 1])
        assert np.array_equal(qi[0], q_all[i]) and si[0] == s_all[i]
    assert np.abs(q_all).max(axis=1).tolist() == [127] * 4


def test_kat_hf_byte_values():
    # packages/inference/tests/test_bitnet_core.py:186-203
    for byte, val in ((0x00, -1), (0x55, 0), (0xAA, 1)):
        assert (O.unpack_hf(np.full((2, 8), byte, np.uint8)) == val).all()


def test_kat_balanced_blocks_times_ones():
    # packages/inference/tests/test_sglang_bitnet.py:111-130: +1 / -1 / 0 column blocks x ones => 0
    t = np.zeros((4, 384), np.int8)
    t[:, :128] = 1
    t[:, 128:256] = -1
    acc = O.int_gemm(np.ones((1, 384), np.int8), t)
    assert not acc.any()


@pytest.mark.parametrize("name", list(gi.CASES))
def test_torch_restatement_of_the_reference_forward(name):
    """oracle/torch_bitlinear.py (the timed "PyTorch BitLinear" CPU baseline) against outputs of the reference's own
    class: same operators in the same order, so fp32 agrees to summation order and bf16 / f16 to one rounding."""
    import torch

    from oracle import torch_bitlinear as TB

    z = np.load(os.path.join(GOLD, f"{name}.npz"))
    x, w = gi.make_inputs(name)
    torch.set_num_threads(1)
    for tag, dt, tol in (("f32", torch.float32, 1e-6), ("bf16", torch.bfloat16, 1e-2), ("f16", torch.float16, 2e-3)):
        y = TB.bitlinear_forward(x.to(dt), w).float().numpy()
        assert np.abs(y - z[f"y_{tag}"]).max() <= tol * np.abs(z[f"y_{tag}"]).max(), tag
    yb = TB.bitlinear_forward(x, w, torch.from_numpy(z["bias"])).numpy()
    assert np.abs(yb - z["y_bias_f32"]).max() <= 1e-6 * np.abs(z["y_bias_f32"]).max()


@pytest.mark.parametrize("tag", ["a", "b"])
def test_oracle_against_bitnet_cpp_goldens(tag):
    """BitNet.cpp's quantize_i2_s / ggml_vec_dot_i2_i8_s outputs (made by its compiled source) against the oracle:
    the I2_S block packing of the sign codes, the uncorrected dot product sum (code * a), and the glue arithmetic
    (dot - sum a) / s_x * s_w (ggml.c:12491-12493)."""
    z = np.load(os.path.join(GOLD, "ggml.npz"))
    w, q = z[f"{tag}_w"], z[f"{tag}_q"]
    t = np.where(np.abs(w.astype(np.float64)) < 1e-6, 0, np.sign(w)).astype(np.int8)
    assert np.array_equal(O.pack_i2s(t), z[f"{tag}_packed"])
    assert np.float32(np.abs(w).max()) == z[f"{tag}_scale"]
    acc = O.int_gemm(q, t)
    sums = q.astype(np.int64).sum(1, keepdims=True)
    assert np.array_equal((acc + sums).astype(np.float32), z[f"{tag}_vec_dot"])
    want = (acc.astype(np.float32) / z[f"{tag}_act_scales"][:, None]) * z[f"{tag}_scale"]
    assert np.allclose(want, z[f"{tag}_mul_mat"], rtol=2e-7, atol=0)
