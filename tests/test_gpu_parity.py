"""GPU parity tests: every CUDA entry point, called through the C ABI, against the CPU
oracle and the golden vectors produced by the reference.  Integer results (codes, int8
activations, int32 accumulators) must be bit-exact; fp32 outputs follow the stated
operation order and must equal the oracle's exactly; outputs are additionally held to
the reference forward within max|a-b|/max|b| <= 1e-5 (fp32) and 1e-2 (bf16 / f16)."""
import os

import numpy as np
import pytest
import torch

import inputs as gi
from oracle import bitlinear_oracle as O

pytestmark = pytest.mark.gpu
GOLD = os.path.join(os.path.dirname(__file__), "golden")
DEV = "cuda:0"
TDT = {"f32": torch.float32, "bf16": torch.bfloat16, "f16": torch.float16}


def load(name):
    z = np.load(os.path.join(GOLD, f"{name}.npz"))
    x, w = gi.make_inputs(name)
    assert gi.sha(x.numpy(), w.numpy()) == str(z["input_sha"])
    return z, x, w


def norm_err(a, b):
    return float(np.abs(a - b).max() / max(np.abs(b).max(), 1e-30))


def test_library_is_loaded_and_device_ok(wf):
    assert wf.check_kernel_available()
    assert wf._lib.lib().wf_version() >= 100


# ---------------------------------------------------------------- weights
@pytest.mark.parametrize("name", list(gi.CASES))
def test_pack_fp32_codes_and_scale(wf, name):
    z, x, w = load(name)
    n, k = w.shape
    codes, scale = wf.pack_ternary(w.to(DEV))
    got = wf.unpack_codes(codes, n, k).cpu().numpy()
    assert np.array_equal(got, z["codes"])  # identical to the reference's own codes
    assert np.array_equal(codes.cpu().numpy(), O.pack_wf16(z["codes"]))  # and to the oracle's packed bytes
    s = scale.cpu().numpy()
    assert s[0] == O.absmean_scale(w.numpy()) and s[1] == s[0]
    # deterministic: a second run gives the same bytes and scale
    codes2, scale2 = wf.pack_ternary(w.to(DEV))
    assert torch.equal(codes, codes2) and torch.equal(scale, scale2)


@pytest.mark.parametrize("name", list(gi.CASES))
@pytest.mark.parametrize("dt", ["bf16", "f16"])
def test_pack_cast_first(wf, name, dt):
    z, x, w = load(name)
    n, k = w.shape
    codes, scale = wf.pack_ternary(w.to(DEV), mode=TDT[dt])
    assert np.array_equal(wf.unpack_codes(codes, n, k).cpu().numpy(), z[f"codes_fwd_{dt}"])
    assert scale.cpu().numpy()[0] == z[f"dequant_fwd_{dt}"]
    # a weight stored in the low-precision type gives the same result
    codes2, scale2 = wf.pack_ternary(w.to(DEV).to(TDT[dt]), mode=TDT[dt])
    assert torch.equal(codes, codes2) and torch.equal(scale, scale2)


def test_pack_edge_cases(wf):
    # all-zero weights -> all-zero codes, scale = eps (test_quantization.py:81-87)
    codes, scale = wf.pack_ternary(torch.zeros(8, 64, device=DEV))
    assert (wf.unpack_codes(codes, 8, 64) == 0).all() and scale[0].item() == np.float32(1e-5)
    # extreme magnitudes stay ternary and finite
    g = torch.Generator().manual_seed(3)
    for mag in (1e-8, 1e6):
        w = torch.randn(16, 128, generator=g) * mag
        codes, scale = wf.pack_ternary(w.to(DEV))
        ref, s = O.ternarize_absmean(w.numpy())
        assert np.array_equal(wf.unpack_codes(codes, 16, 128).cpu().numpy(), ref) and scale[0].item() == s
    # strided rows
    w = torch.randn(16, 256, generator=g) * 0.02
    wide = torch.zeros(16, 320)
    wide[:, :256] = w
    c1, s1 = wf.pack_ternary(w.to(DEV))
    c2, s2 = wf.pack_ternary(wide.to(DEV)[:, :256])
    assert torch.equal(c1, c2) and torch.equal(s1, s2)
    with pytest.raises(RuntimeError):
        wf.pack_ternary(torch.zeros(4, 48, device=DEV))  # K % 64 != 0


def test_layout_conversions(wf):
    z = np.load(os.path.join(GOLD, "packers.npz"))
    t = z["ternary"]
    n, k = t.shape
    L = wf._lib
    want_wf16, want_i2s = O.pack_wf16(t), O.pack_i2s(t)
    tt = torch.from_numpy(t).to(DEV)
    assert np.array_equal(wf.pack_codes(tt, L.LAYOUT_WF16).cpu().numpy(), want_wf16)
    assert np.array_equal(wf.pack_codes(tt, L.LAYOUT_I2S).cpu().numpy(), want_i2s)
    assert np.array_equal(want_i2s, z["sglkernel_simd"])  # the reference packer's own bytes
    srcs = {L.LAYOUT_I2S: z["sglkernel_simd"], L.LAYOUT_SEQ_LSB: z["native_seq_lsb"],
            L.LAYOUT_SEQ_MSB: z["quantize_to_bitnet_msb"], L.LAYOUT_HF: O.pack_hf(t), L.LAYOUT_WF16: want_wf16}
    for lay, src in srcs.items():
        s = torch.from_numpy(np.ascontiguousarray(src)).to(DEV)
        assert np.array_equal(wf.repack(s, lay, n, k, L.LAYOUT_WF16).cpu().numpy(), want_wf16), lay
        assert np.array_equal(wf.repack(s, lay, n, k, L.LAYOUT_I2S).cpu().numpy(), want_i2s), lay
        assert np.array_equal(wf.unpack_codes(s, n, k, lay).cpu().numpy(), t), lay
    # the HF bytes the reference's unpacker was pinned on
    hf = torch.from_numpy(z["hf_bytes"]).to(DEV)
    assert np.array_equal(wf.unpack_codes(hf, 16, 256, L.LAYOUT_HF).cpu().numpy(), z["hf_unpacked"])


# ---------------------------------------------------------------- activations
@pytest.mark.parametrize("name", list(gi.CASES))
@pytest.mark.parametrize("dt", ["f32", "bf16", "f16"])
def test_act_quant_per_token(wf, name, dt):
    z, x, w = load(name)
    q, s, rs = wf.act_quant_i8(x.to(TDT[dt]).to(DEV), want_rowsum=True)
    assert np.array_equal(q.cpu().numpy(), z[f"q_{dt}"])
    assert np.array_equal(s.cpu().numpy(), z[f"act_scale_{dt}"])
    assert np.array_equal(rs.cpu().numpy(), z[f"q_{dt}"].astype(np.int32).sum(1))


@pytest.mark.parametrize("name", gi.I2S_CASES)
def test_act_quant_per_tensor(wf, name):
    z, x, w = load(name)
    q, s = wf.quantize_activations_i8(x.to(DEV))
    assert np.array_equal(q.cpu().numpy(), z["i2s_q_tensor"])
    assert s.cpu().numpy()[0] == z["i2s_act_scale"]
    q0, s0 = wf.quantize_activations_i8(torch.zeros(2, 64, device=DEV))
    assert not q0.any() and s0.item() == np.float32(1.0 / 127.0)


def test_act_quant_edge_cases(wf):
    g = torch.Generator().manual_seed(4)
    x = torch.randn(7, 256, generator=g)
    x[2] = 0  # all-zero token: absmax clamps to eps
    x[3] *= 1000.0
    x[4] *= 1e-6
    for dt in ("f32", "bf16"):
        xd = x.to(TDT[dt])
        q, s = wf.act_quant_i8(xd.to(DEV))
        qo, so = O.act_quant_per_token(xd.float().numpy(), dt)
        assert np.array_equal(q.cpu().numpy(), qo) and np.array_equal(s.cpu().numpy(), so)


@pytest.mark.parametrize("k", [72, 2560, 6912, 16384])
@pytest.mark.parametrize("dt", ["f32", "bf16", "f16"])
def test_act_quant_many_tokens(wf, k, dt):
    """A few hundred tokens of the widths the sweep uses (and one beyond): codes, multipliers and row sums equal the
    oracle's, outliers, an all-zero token and a strided view included."""
    g = torch.Generator().manual_seed(k)
    m = 203
    x = gi.with_outliers(torch.randn(m, k, generator=g), seed=k)
    x[5] = 0
    x[6] *= 1e-3 if dt == "f16" else 1e-6  # small against eps, still a normal number in every type
    xd = x.to(TDT[dt])
    q, s, rs = wf.act_quant_i8(xd.to(DEV), want_rowsum=True)
    qo, so = O.act_quant_per_token(xd.float().numpy(), dt)
    assert np.array_equal(q.cpu().numpy(), qo) and np.array_equal(s.cpu().numpy(), so)
    assert np.array_equal(rs.cpu().numpy(), qo.astype(np.int32).sum(1))
    # a strided view: rows of a wider buffer
    wide = torch.zeros(m, k + 24, dtype=TDT[dt])
    wide[:, :k] = xd
    q2, s2 = wf.act_quant_i8(wide.to(DEV)[:, :k])
    assert torch.equal(q2, q) and torch.equal(s2, s)


# ---------------------------------------------------------------- contraction
@pytest.mark.parametrize("name", list(gi.CASES))
@pytest.mark.parametrize("dt", ["f32", "bf16", "f16"])
def test_decode_against_golden(wf, name, dt):
    z, x, w = load(name)
    codes, scale = wf.pack_ternary(w.to(DEV))
    xd = x.to(TDT[dt])
    y, acc = wf.bitlinear(xd.to(DEV), codes, scale, out_dtype=torch.float32, want_acc=True)
    acc_o = O.int_gemm(z[f"q_{dt}"], z["codes"])
    assert np.array_equal(acc.cpu().numpy(), acc_o)  # int32 accumulators: bit-exact
    y_o = O.rescale(acc_o, z[f"act_scale_{dt}"], O.absmean_scale(w.numpy()))
    assert np.array_equal(y.cpu().numpy(), y_o)  # same fp32 operation order -> identical
    if dt == "f32":
        assert norm_err(y.cpu().numpy(), z["y_f32"]) < 1e-5
        yb = wf.bitlinear(xd.to(DEV), codes, scale, bias=torch.from_numpy(z["bias"]).to(DEV))
        assert norm_err(yb.cpu().numpy(), z["y_bias_f32"]) < 1e-5
    else:
        # against the low-precision reference forward the weights are packed the way that forward forms them
        codes_c, scale_c = wf.pack_ternary(w.to(DEV), mode=TDT[dt])
        yc = wf.bitlinear(xd.to(DEV), codes_c, scale_c)
        assert yc.dtype == TDT[dt]
        assert norm_err(yc.float().cpu().numpy(), z[f"y_{dt}"]) < 1e-2


SHAPES = [  # (M, K, N)
    (1, 64, 16), (2, 128, 24), (3, 192, 40), (4, 576, 100), (5, 640, 16), (7, 1024, 33), (8, 2560, 64), (9, 512, 48),
    (16, 576, 1536), (17, 1088, 80), (33, 2560, 96), (64, 2560, 160), (64, 6912, 64), (70, 640, 32), (1, 6912, 2560),
    (4, 2560, 6912), (1, 4096, 14336), (130, 256, 48), (32, 14336, 64), (9, 16384, 32),
]


@pytest.mark.parametrize("m,k,n", SHAPES)
def test_decode_random_shapes_bit_exact(wf, oracle_c, m, k, n):
    rng = np.random.default_rng(m * 100003 + k * 17 + n)
    t = rng.integers(-1, 2, size=(n, k)).astype(np.int8)
    x = torch.from_numpy(rng.standard_normal((m, k)).astype(np.float32))
    x = gi.with_outliers(x, seed=m + k + n)
    L = wf._lib
    for dt in ("bf16", "f32"):
        xd = x.to(TDT[dt])
        q, s = oracle_c.act_quant(xd.float().numpy(), {"f32": 0, "bf16": 1}[dt])
        acc_o = oracle_c.int_gemm(q, t)
        y_o = oracle_c.rescale(acc_o, s, 0.0173)
        for lay in ((L.LAYOUT_WF16, L.LAYOUT_I2S) if k % 128 == 0 else (L.LAYOUT_WF16,)):
            codes = wf.pack_codes(torch.from_numpy(t).to(DEV), lay)
            y, acc = wf.bitlinear(xd.to(DEV), codes, 0.0173, layout=lay, out_dtype=torch.float32, want_acc=True,
                                  path="decode")
            assert np.array_equal(acc.cpu().numpy(), acc_o), (dt, lay)
            assert np.array_equal(y.cpu().numpy(), y_o), (dt, lay)


def test_decode_extreme_codes_and_activations(wf):
    """All 81 four-code combinations against activations pinned at -128 and 127."""
    k = 64
    combos = np.array([[a, b, c, d] for a in (-1, 0, 1) for b in (-1, 0, 1) for c in (-1, 0, 1) for d in (-1, 0, 1)], np.int8)
    t = np.tile(combos, (1, k // 4))  # [81, 64]
    q = np.empty((4, k), np.int8)
    q[0], q[1] = 127, -128
    q[2] = np.where(np.arange(k) % 2 == 0, 127, -128)
    q[3] = np.where(np.arange(k) % 3 == 0, -128, 127)
    codes = wf.pack_codes(torch.from_numpy(t).to(DEV))
    y, acc = wf.bitlinear(torch.from_numpy(q).to(DEV), codes, 1.0, want_acc=True)
    assert np.array_equal(acc.cpu().numpy(), O.int_gemm(q, t))
    assert np.array_equal(y.cpu().numpy(), O.int_gemm(q, t).astype(np.float32))


def test_int8_input_with_scales_and_strides(wf):
    rng = np.random.default_rng(9)
    m, k, n = 6, 384, 50
    t = rng.integers(-1, 2, size=(n, k)).astype(np.int8)
    q = rng.integers(-128, 128, size=(m, k)).astype(np.int8)
    s = (rng.random(m).astype(np.float32) + 0.5) * 40
    codes = wf.pack_codes(torch.from_numpy(t).to(DEV))
    wide = torch.zeros(m, k + 64, dtype=torch.int8, device=DEV)
    wide[:, :k] = torch.from_numpy(q).to(DEV)
    out = torch.empty(m, n + 14, device=DEV)[:, :n]
    ws = torch.tensor([0.021], device=DEV)
    y, acc = wf.bitlinear(wide[:, :k], codes, ws, x_scale=torch.from_numpy(s).to(DEV), want_acc=True, out=None)
    acc_o = O.int_gemm(q, t)
    assert np.array_equal(acc.cpu().numpy(), acc_o)
    assert np.array_equal(y.cpu().numpy(), O.rescale(acc_o, s, np.float32(0.021)))


def test_prefill_entry_point_bit_exact(wf, oracle_c):
    """The tensor-core contraction: partial token / row / K tiles, both layouts, float and int8 input, bias."""
    L = wf._lib
    rng = np.random.default_rng(21)
    for (m, k, n) in ((128, 256, 64), (200, 576, 144), (512, 2560, 256), (300, 1024, 700), (129, 128, 257)):
        t = rng.integers(-1, 2, size=(n, k)).astype(np.int8)
        x = torch.from_numpy(rng.standard_normal((m, k)).astype(np.float32)).bfloat16()
        bias = torch.from_numpy(rng.standard_normal(n).astype(np.float32))
        q, s = oracle_c.act_quant(x.float().numpy(), 1)
        acc_o = oracle_c.int_gemm(q, t)
        for lay in ((L.LAYOUT_WF16, L.LAYOUT_I2S) if k % 128 == 0 else (L.LAYOUT_WF16,)):
            codes = wf.pack_codes(torch.from_numpy(t).to(DEV), lay)
            y, acc = wf.bitlinear(x.to(DEV), codes, 0.02, layout=lay, out_dtype=torch.float32, want_acc=True, path="prefill")
            assert np.array_equal(acc.cpu().numpy(), acc_o), (m, k, n, lay)
            assert np.array_equal(y.cpu().numpy(), oracle_c.rescale(acc_o, s, 0.02))
        yb = wf.bitlinear(x.to(DEV), codes, 0.02, bias=bias.to(DEV), layout=lay, out_dtype=torch.float32, path="prefill")
        assert np.array_equal(yb.cpu().numpy(), oracle_c.rescale(acc_o, s, 0.02, bias.numpy()))
        # already-quantized input with per-token multipliers
        yq, accq = wf.bitlinear(torch.from_numpy(q).to(DEV), codes, 0.02, layout=lay, x_scale=torch.from_numpy(s).to(DEV),
                                want_acc=True, path="prefill")
        assert np.array_equal(accq.cpu().numpy(), acc_o) and np.array_equal(yq.cpu().numpy(), oracle_c.rescale(acc_o, s, 0.02))
    wf.device_status()


def test_small_m_contraction_bit_exact(wf, oracle_c):
    """Up to 64 tokens the contraction swaps the operand roles (128 weight rows x 16/32/64 tokens, expanded weights in
    tensor memory): partial row blocks, K tails (also a packed stage of a single K block), both layouts, bias, int8 input."""
    L = wf._lib
    rng = np.random.default_rng(23)
    for (m, k, n) in ((1, 256, 64), (16, 576, 144), (17, 1024, 700), (33, 2560, 256), (64, 128, 257), (40, 6912, 300),
                      (5, 640, 130), (64, 1664, 128)):
        t = rng.integers(-1, 2, size=(n, k)).astype(np.int8)
        x = torch.from_numpy(rng.standard_normal((m, k)).astype(np.float32)).bfloat16()
        bias = torch.from_numpy(rng.standard_normal(n).astype(np.float32))
        q, s = oracle_c.act_quant(x.float().numpy(), 1)
        acc_o = oracle_c.int_gemm(q, t)
        for lay in ((L.LAYOUT_WF16, L.LAYOUT_I2S) if k % 128 == 0 else (L.LAYOUT_WF16,)):
            codes = wf.pack_codes(torch.from_numpy(t).to(DEV), lay)
            y, acc = wf.bitlinear(x.to(DEV), codes, 0.02, layout=lay, out_dtype=torch.float32, want_acc=True, path="prefill")
            assert np.array_equal(acc.cpu().numpy(), acc_o), (m, k, n, lay)
            assert np.array_equal(y.cpu().numpy(), oracle_c.rescale(acc_o, s, 0.02)), (m, k, n, lay)
        yb = wf.bitlinear(x.to(DEV), codes, 0.02, bias=bias.to(DEV), layout=lay, path="prefill")
        assert yb.dtype == torch.bfloat16
        want = torch.from_numpy(oracle_c.rescale(acc_o, s, 0.02, bias.numpy())).bfloat16()
        assert torch.equal(yb.cpu(), want), (m, k, n)
        yq, accq = wf.bitlinear(torch.from_numpy(q).to(DEV), codes, 0.02, layout=lay, x_scale=torch.from_numpy(s).to(DEV),
                                want_acc=True, path="prefill")
        assert np.array_equal(accq.cpu().numpy(), acc_o) and np.array_equal(yq.cpu().numpy(), oracle_c.rescale(acc_o, s, 0.02))
    wf.device_status()


def test_prefill_pair_form_bit_exact(wf, oracle_c):
    """The two-SM form of the contraction (a cluster of two CTAs per 256-row x 192-token tile, tcgen05 cta_group::2):
    partial token blocks, partial row blocks (also a tile whose second CTA has no valid row), K tails inside and
    across the 512-wide packed stages, several tiles per cluster, both layouts, bias, int8 input; and the forced
    single-SM form on the same data."""
    L = wf._lib
    rng = np.random.default_rng(29)
    for (m, k, n) in ((192, 256, 256), (65, 128, 100), (200, 576, 300), (385, 1024, 700), (500, 2560, 520), (129, 128, 257),
                      (70, 6912, 256), (3000, 640, 9000)):
        t = rng.integers(-1, 2, size=(n, k)).astype(np.int8)
        x = torch.from_numpy(rng.standard_normal((m, k)).astype(np.float32)).bfloat16()
        bias = torch.from_numpy(rng.standard_normal(n).astype(np.float32))
        q, s = oracle_c.act_quant(x.float().numpy(), 1)
        acc_o = oracle_c.int_gemm(q, t)
        y_o = oracle_c.rescale(acc_o, s, 0.02)
        for lay in ((L.LAYOUT_WF16, L.LAYOUT_I2S) if k % 128 == 0 else (L.LAYOUT_WF16,)):
            codes = wf.pack_codes(torch.from_numpy(t).to(DEV), lay)
            for form in ("pair", "single"):
                y, acc = wf.bitlinear(x.to(DEV), codes, 0.02, layout=lay, out_dtype=torch.float32, want_acc=True, path="prefill",
                                      prefill_form=form)
                assert np.array_equal(acc.cpu().numpy(), acc_o), (m, k, n, lay, form)
                assert np.array_equal(y.cpu().numpy(), y_o), (m, k, n, lay, form)
        yb = wf.bitlinear(x.to(DEV), codes, 0.02, bias=bias.to(DEV), layout=lay, path="prefill", prefill_form="pair")
        want = torch.from_numpy(oracle_c.rescale(acc_o, s, 0.02, bias.numpy())).bfloat16()
        assert yb.dtype == torch.bfloat16 and torch.equal(yb.cpu(), want), (m, k, n)
        yq, accq = wf.bitlinear(torch.from_numpy(q).to(DEV), codes, 0.02, layout=lay, x_scale=torch.from_numpy(s).to(DEV),
                                want_acc=True, path="prefill", prefill_form="pair")
        assert np.array_equal(accq.cpu().numpy(), acc_o) and np.array_equal(yq.cpu().numpy(), y_o)
        wf.device_status()


@pytest.mark.parametrize("n,k", [(2560, 2560), (6912, 2560), (2560, 6912)])
def test_prefill_full_size_against_decode_path(wf, n, k):
    """BASELINE prefill shapes at M = 512: the tensor-core path and the decode path agree bit for bit."""
    g = torch.Generator().manual_seed(n + k)
    w = torch.randn(n, k, generator=g) * 0.02
    x = gi.with_outliers(torch.randn(512, k, generator=g), seed=3).bfloat16().to(DEV)
    codes, scale = wf.pack_ternary(w.to(DEV))
    y1, a1 = wf.bitlinear(x, codes, scale, want_acc=True, path="prefill")
    y2, a2 = wf.bitlinear(x, codes, scale, want_acc=True, path="decode")
    assert torch.equal(a1, a2) and torch.equal(y1, y2)
    wf.device_status()


# ---------------------------------------------------------------- operator API and modules
@pytest.mark.parametrize("name", gi.I2S_CASES)
def test_operator_api_matches_reference_kernel(wf, name):
    z, x, w = load(name)
    m, k, n, _ = gi.CASES[name]
    packed = torch.from_numpy(O.pack_i2s(z["codes"])).to(DEV)
    q, s = wf.quantize_activations_i8(x.to(DEV))
    out = wf.bitnet_gemm(packed, q, float(z["w_scale_torch"]))
    assert out.dtype == torch.float32 and tuple(out.shape) == (m, n)
    assert np.array_equal(out.cpu().numpy(), z["i2s_gemm"])  # the compiled reference kernel's own output
    v = wf.bitnet_gemv(packed, q[0], float(z["w_scale_torch"]))
    assert np.array_equal(v.cpu().numpy(), z["i2s_gemv_row0"])
    with pytest.raises(ValueError):
        wf.bitnet_gemv(packed[:, :16], q[0, :64], 1.0)  # K % 128 != 0, as the reference rejects


@pytest.mark.parametrize("dt", ["f32", "bf16", "f16"])
def test_bitlinear_module_drop_in(wf, dt):
    z, x, w = load("c1")
    layer = wf.BitLinear(576, 1536, bias=False).to(DEV)
    with torch.no_grad():
        layer.weight.copy_(w.to(DEV))
        y = layer(x.to(TDT[dt]).to(DEV).reshape(2, 8, 576))
    assert y.dtype == TDT[dt] and tuple(y.shape) == (2, 8, 1536)
    tol = 1e-5 if dt == "f32" else 1e-2
    assert norm_err(y.float().cpu().numpy().reshape(16, 1536), z[f"y_{dt}"]) < tol
    # weight update invalidates the packed copy
    with torch.no_grad():
        layer.weight.mul_(2.0)
        y2 = layer(x.to(TDT[dt]).to(DEV))
    assert norm_err(y2.float().cpu().numpy(), 2 * z[f"y_{dt}"]) < max(tol, 4e-3 if dt != "f32" else 0)
    with pytest.raises(RuntimeError):
        with torch.no_grad():
            layer(x)  # CPU tensor: no fallback


def test_bitlinear_module_training_formula_on_gpu(wf):
    z, x, w = load("k192")
    layer = wf.BitLinear(192, 80).to(DEV)
    with torch.no_grad():
        layer.weight.copy_(w.to(DEV))
    xg = x.to(DEV).requires_grad_(True)
    y = layer(xg)  # gradient needed -> straight-through formula
    y.sum().backward()
    assert xg.grad is not None and layer.weight.grad is not None
    assert norm_err(y.detach().cpu().numpy(), z["y_f32"]) < 1e-5
    with torch.no_grad():
        y_fast = layer(x.to(DEV))
    assert norm_err(y_fast.cpu().numpy(), y.detach().cpu().numpy()) < 1e-5


def test_linear_methods(wf):
    z, x, w = load("k512")
    m, k, n, _ = gi.CASES["k512"]
    packed = torch.from_numpy(O.pack_i2s(z["codes"])).to(DEV)
    scale = torch.tensor([float(z["w_scale_torch"])], device=DEV)
    method = wf.BitNetConfig().get_quant_method(None, "")
    layer = torch.nn.Module()
    method.create_weights(layer, k, [n], k, n, torch.bfloat16)
    assert tuple(layer.qweight.shape) == (n, k // 4) and layer.qweight.pack_factor == 4
    layer = layer.to(DEV)
    layer.qweight.data.copy_(packed)
    layer.scale.data.copy_(scale)
    method.process_weights_after_loading(layer)
    out = method.apply(layer, x.to(DEV))
    assert out.dtype == torch.float32
    assert norm_err(out.cpu().numpy(), z["y_f32"]) < 1e-5
    # the reference's own per-tensor arithmetic, as its apply() composes it
    pt = wf.BitNetLinearMethod(wf.BitNetConfig(act_quant="per_tensor")).apply(layer, x.to(DEV))
    assert norm_err(pt.cpu().numpy(), z["i2s_gemm"] * z["i2s_act_scale"]) < 1e-6
    with pytest.raises(ValueError):
        method.create_weights(torch.nn.Module(), 576, [64], 576, 64, torch.bfloat16)  # K % 128 != 0
    fp = wf.PackedBitNetLinearMethod(layout=wf._lib.LAYOUT_I2S).apply(packed, scale, x.to(DEV).bfloat16(), n, k)
    assert fp.dtype == torch.bfloat16 and norm_err(fp.float().cpu().numpy(), z["y_f32"]) < 2e-2
    nat = wf.BitNetLinearNative(k, n, packed, scale, layout=wf._lib.LAYOUT_I2S)(x.to(DEV))
    assert norm_err(nat.cpu().numpy(), z["y_f32"]) < 1e-5


# ---------------------------------------------------------------- BASELINE sizes: properties
@pytest.mark.parametrize("n,k", [(2560, 2560), (6912, 2560), (2560, 6912)])
@pytest.mark.parametrize("m", [1, 4, 16, 64])
def test_full_size_sweep_properties(wf, oracle_c, n, k, m):
    g = torch.Generator().manual_seed(1000 * (n // 1000) + m)
    w = torch.randn(n, k, generator=g) * 0.02
    x = gi.with_outliers(torch.randn(m, k, generator=g), seed=m).bfloat16()
    codes, scale = wf.pack_ternary(w.to(DEV))
    zero_frac = float((wf.unpack_codes(codes, n, k) == 0).float().mean())
    assert 0.29 < zero_frac < 0.33  # about 31 % zeros for absmean-ternarized Gaussians
    y, acc = wf.bitlinear(x.to(DEV), codes, scale, out_dtype=torch.float32, want_acc=True)
    # a slice of rows against the oracle, bit-exact
    rows = slice(0, n, max(1, n // 64))
    t, s_w = O.ternarize_absmean(w.numpy()[rows])
    q, s = oracle_c.act_quant(x.float().numpy(), 1)
    t_rows = wf.unpack_codes(codes, n, k).cpu().numpy()[rows]
    assert np.array_equal(acc.cpu().numpy()[:, rows], oracle_c.int_gemm(q, t_rows))
    # checksum over all rows: sum_n acc[m, n] = q[m] . (sum_n codes[n])
    colsum = wf.unpack_codes(codes, n, k).to(torch.int64).sum(0).cpu().numpy()
    assert np.array_equal(acc.to(torch.int64).sum(1).cpu().numpy(), q.astype(np.int64) @ colsum)
    # linearity in the weights' sign: negated codes negate the accumulators
    neg = wf.pack_codes(-wf.unpack_codes(codes, n, k))
    _, acc_neg = wf.bitlinear(x.to(DEV), neg, scale, out_dtype=torch.float32, want_acc=True)
    assert torch.equal(acc_neg, -acc)
    # determinism
    y2 = wf.bitlinear(x.to(DEV), codes, scale, out_dtype=torch.float32)
    assert torch.equal(y, y2)


@pytest.mark.parametrize("m", [1, 8, 20])
def test_decode_many_items_per_cta_equals_contraction(wf, m):
    """A single tall matrix (more 16-row items per CTA than ring stages) and a gate/up-like pair on shared tokens: the
    decode kernel lets every warp take whole items there; results must equal the tensor-core path bit for bit."""
    g = torch.Generator().manual_seed(900 + m)
    n, k = 65536, 512  # 4096 items: about 28 per CTA, more than the ring has stages
    w = torch.randn(n, k, generator=g) * 0.02
    x = gi.with_outliers(torch.randn(m, k, generator=g), seed=4).bfloat16().to(DEV)
    codes, scale = wf.pack_ternary(w.to(DEV))
    y1, a1 = wf.bitlinear(x, codes, scale, want_acc=True, path="decode")
    y2, a2 = wf.bitlinear(x, codes, scale, want_acc=True, path="prefill")
    assert torch.equal(a1, a2) and torch.equal(y1, y2)
    half = n // 2
    grp = wf.DecodeGroup([dict(x=x, codes=codes[:half].contiguous(), w_scale=scale, want_acc=True),
                          dict(x=x, codes=codes[half:].contiguous(), w_scale=scale, want_acc=True)])
    for rep in range(2):
        outs = grp.run(pdl=bool(rep))
        assert torch.equal(torch.cat(grp.accs, 1), a2) and torch.equal(torch.cat(outs, 1), y2)
    wf.device_status()


# ---------------------------------------------------------------- grouped launches
def test_grouped_decode_matches_single_calls(wf, oracle_c):
    """q/k/v-like and mixed-shape groups: one persistent launch, results identical to the oracle."""
    rng = np.random.default_rng(77)
    specs = [(3, 256, 96), (3, 256, 32), (3, 256, 32), (5, 576, 100), (1, 2560, 2560), (8, 640, 48), (2, 128, 16)]
    probs, want = [], []
    for (m, k, n) in specs:
        t = rng.integers(-1, 2, size=(n, k)).astype(np.int8)
        x = torch.from_numpy(rng.standard_normal((m, k)).astype(np.float32)).bfloat16()
        q, s = oracle_c.act_quant(x.float().numpy(), 1)
        acc = oracle_c.int_gemm(q, t)
        want.append((acc, oracle_c.rescale(acc, s, 0.02)))
        probs.append(dict(x=x.to(DEV), codes=wf.pack_codes(torch.from_numpy(t).to(DEV)), w_scale=0.02,
                          out_dtype=torch.float32, want_acc=True))
    grp = wf.DecodeGroup(probs)
    for rep in range(2):  # the descriptor array is reusable
        outs = grp.run(pdl=bool(rep))
        for y, acc, (acc_o, y_o) in zip(outs, grp.accs, want):
            assert np.array_equal(acc.cpu().numpy(), acc_o)
            assert np.array_equal(y.cpu().numpy(), y_o)
    wf.device_status()


def test_grouped_large_stack(wf, oracle_c):
    """A stack of layers larger than one wave of CTAs, M > token tile (several passes)."""
    rng = np.random.default_rng(78)
    probs, want = [], []
    for i in range(12):
        m, k, n = (20 if i % 2 else 1), 1024, 1000 + 16 * i
        t = rng.integers(-1, 2, size=(n, k)).astype(np.int8)
        x = torch.from_numpy(rng.standard_normal((m, k)).astype(np.float32))
        q, s = oracle_c.act_quant(x.numpy(), 0)
        acc = oracle_c.int_gemm(q, t)
        want.append(acc)
        probs.append(dict(x=x.to(DEV), codes=wf.pack_codes(torch.from_numpy(t).to(DEV)), w_scale=1.0, want_acc=True))
    grp = wf.DecodeGroup(probs)
    grp.run()
    for acc, acc_o in zip(grp.accs, want):
        assert np.array_equal(acc.cpu().numpy(), acc_o)
    wf.device_status()


@pytest.mark.parametrize("m,dt", [(1, "bf16"), (4, "f32"), (16, "bf16"), (40, "bf16")])
def test_grouped_throughput_mode_equals_single_calls(wf, oracle_c, m, dt):
    """Groups with thousands of 16-row items take the form of the kernel in which every warp consumes
    its own items; accumulators and outputs must equal those of single calls (and the oracle's)."""
    L = wf._lib
    rng = np.random.default_rng(500 + m)
    shapes = [(4000, 1024), (6912, 2560), (2560, 6912), (3000, 576), (5000, 640), (6000, 1024), (6912, 1280), (4096, 2048)]
    probs, singles = [], []
    for i, (n, k) in enumerate(shapes):
        lay = L.LAYOUT_I2S if (i % 2 and k % 128 == 0) else L.LAYOUT_WF16
        t = torch.from_numpy(rng.integers(-1, 2, size=(n, k)).astype(np.int8)).to(DEV)
        codes = wf.pack_codes(t, lay)
        x = gi.with_outliers(torch.from_numpy(rng.standard_normal((m, k)).astype(np.float32)), seed=i).to(TDT[dt]).to(DEV)
        bias = torch.from_numpy(rng.standard_normal(n).astype(np.float32)).to(DEV) if i % 3 == 0 else None
        probs.append(dict(x=x, codes=codes, w_scale=0.0173, bias=bias, layout=lay, out_dtype=torch.float32, want_acc=True))
        singles.append(wf.bitlinear(x, codes, 0.0173, bias=bias, layout=lay, out_dtype=torch.float32, want_acc=True,
                                    path="decode"))
        if i == 0:  # one of them against the CPU oracle directly
            q, s = oracle_c.act_quant(x.float().cpu().numpy(), {"f32": 0, "bf16": 1}[dt])
            assert np.array_equal(singles[0][1].cpu().numpy(), oracle_c.int_gemm(q, t.cpu().numpy()))
    grp = wf.DecodeGroup(probs)
    # plain launch; chained launches with a programmatic dependency; the same with inputs declared ready (the kernel
    # then reads x before it waits for the previous launch, and only its stores wait)
    for rep, (pdl, x_ready) in enumerate([(False, False), (True, False), (True, True), (True, True)]):
        for a in grp.accs:
            a.fill_(-7)
        outs = grp.run(pdl=pdl, x_ready=x_ready)
        for (y1, a1), y2, a2 in zip(singles, outs, grp.accs):
            assert torch.equal(a1, a2), (rep, pdl, x_ready)
            assert torch.equal(y1, y2), (rep, pdl, x_ready)
    wf.device_status()


def test_batched_prefill_equals_per_layer_calls(wf, oracle_c):
    """Stacked layers in one tensor-core launch: every layer's accumulators equal the oracle's."""
    rng = np.random.default_rng(91)
    for (b, m, k, n) in ((3, 64, 512, 200), (5, 16, 576, 256), (2, 130, 256, 300)):
        t = rng.integers(-1, 2, size=(b, n, k)).astype(np.int8)
        x = torch.from_numpy(rng.standard_normal((b, m, k)).astype(np.float32)).bfloat16()
        codes = torch.stack([wf.pack_codes(torch.from_numpy(t[i]).to(DEV)) for i in range(b)]).contiguous()
        scales = torch.tensor([[0.01 * (i + 1), 0.0] for i in range(b)], device=DEV)
        y, acc = wf.bitlinear_batched(x.to(DEV), codes, scales, out_dtype=torch.float32, want_acc=True)
        for i in range(b):
            q, s = oracle_c.act_quant(x[i].float().numpy(), 1)
            acc_o = oracle_c.int_gemm(q, t[i])
            assert np.array_equal(acc[i].cpu().numpy(), acc_o), (b, m, k, n, i)
            assert np.array_equal(y[i].cpu().numpy(), oracle_c.rescale(acc_o, s, np.float32(0.01 * (i + 1))))
    wf.device_status()


# ---------------------------------------------------------------- training step on the packed weights
@pytest.mark.parametrize("dt,tol", [("f32", 1e-5), ("bf16", 2e-2)])
def test_training_step_on_packed_weights(wf, dt, tol):
    """With gradients enabled at lambda = 1 the module runs the packed forward inside a straight-through autograd
    function.  Its output and its gradients are held to the reference's own formula
    (F.linear(x + (aq(x) - x).detach(), w + (wq(w) - w).detach(), b), bitlinear.py:99-113) evaluated by autograd on
    the same tensors; an optimizer step must invalidate the cached codes (test_paper_verification.py:302-381 checks
    the same properties of the reference: gradients reach x, weight and bias and are non-zero)."""
    z, x, w = load("k512")
    m, k, n, _ = gi.CASES["k512"]
    tdt = TDT[dt]
    g = torch.Generator().manual_seed(17)
    bias0 = torch.randn(n, generator=g) * 0.1
    dy = torch.randn(2, m // 2, n, generator=g).to(tdt).to(DEV)
    layer = wf.BitLinear(k, n, bias=True).to(DEV)
    with torch.no_grad():
        layer.weight.copy_(w.to(DEV))
        layer.bias.copy_(bias0.to(DEV))
    xg = x.to(tdt).to(DEV).reshape(2, m // 2, k).requires_grad_(True)
    y = layer(xg)
    assert y.grad_fn is not None and "PackedSTE" in type(y.grad_fn).__name__ and y.dtype == tdt
    y.backward(dy)
    # the reference formula on the same tensors
    xr = x.to(tdt).to(DEV).reshape(2, m // 2, k).requires_grad_(True)
    wr = layer.weight.detach().clone().requires_grad_(True)
    br = layer.bias.detach().clone().requires_grad_(True)
    wl = wr.to(tdt)
    w_quant = wl + (layer.weight_quant(wl) - wl).detach()
    x_quant = xr + (layer.activation_quant(xr) - xr).detach()
    y_ref = torch.nn.functional.linear(x_quant, w_quant, br.to(tdt))
    y_ref.backward(dy)

    def rel(a, b):
        return float((a.float() - b.float()).abs().max() / b.float().abs().max())

    assert rel(y, y_ref) <= (1e-5 if dt == "f32" else 1e-2)
    assert rel(xg.grad, xr.grad) <= tol and rel(layer.weight.grad, wr.grad) <= tol and rel(layer.bias.grad, br.grad) <= tol
    assert layer.weight.grad.dtype == layer.weight.dtype and float(xg.grad.abs().sum()) > 0
    # an optimizer step changes the weight: the next forward must re-pack
    codes_before = layer.packed_weight(tdt)[0].clone()
    opt = torch.optim.SGD(layer.parameters(), lr=0.5)
    opt.step()
    y2 = layer(xg.detach())
    codes_after = layer.packed_weight(tdt)[0]
    assert not torch.equal(codes_before, codes_after)
    with torch.no_grad():
        want = torch.nn.functional.linear(layer.activation_quant(xg.detach()), layer.weight_quant(layer.weight.to(tdt)), layer.bias.to(tdt))
    assert rel(y2, want) <= (1e-5 if dt == "f32" else 1e-2)
    # during the lambda warm-up the module evaluates the reference's mixing formula
    warm = wf.LambdaWarmup(warmup_steps=4)
    wf.set_global_lambda_warmup(warm)
    try:
        warm.step()
        warm.step()  # lambda = 0.5
        y3 = layer(xg)
        assert "PackedSTE" not in type(y3.grad_fn).__name__
        wl2 = layer.weight.to(tdt)
        want3 = torch.nn.functional.linear(xg + 0.5 * (layer.activation_quant(xg) - xg), wl2 + 0.5 * (layer.weight_quant(wl2) - wl2), layer.bias.to(tdt))
        assert rel(y3, want3) <= 1e-6
    finally:
        wf.set_global_lambda_warmup(None)


@pytest.mark.parametrize("k", [64, 512, 1024, 1536, 2560])
@pytest.mark.parametrize("m", [16, 24, 32, 33, 64])
def test_few_token_contraction_stage_counts(wf, k, m):
    """The few-token forms of the contraction share the K stages out among two or three issuing threads with partial
    accumulators: every count of stages per tile (fewer than issuing threads, equal, more, not a multiple), one layer
    and a stack, against the decode kernel's outputs bit for bit (both are held to the oracle elsewhere)."""
    g = torch.Generator(device=DEV).manual_seed(k + m)
    n = 384
    for layers in (1, 5):
        codes = torch.empty(layers, n, k // 4, dtype=torch.uint8, device=DEV)
        scales = torch.empty(layers, 2, device=DEV)
        for i in range(layers):
            c, s = wf.pack_ternary(torch.randn(n, k, generator=g, device=DEV) * 0.02)
            codes[i].copy_(c)
            scales[i].copy_(s)
        x = torch.randn(layers, m, k, generator=g, device=DEV).bfloat16()
        y = torch.empty(layers, m, n, dtype=torch.float32, device=DEV)
        wf.bitlinear_batched(x, codes, scales, out=y)
        for i in range(layers):
            assert torch.equal(wf.bitlinear(x[i], codes[i], scales[i], out_dtype=torch.float32, path="decode"), y[i]), (layers, i)
    wf.device_status()


@pytest.mark.parametrize("m", [16, 64, 200])
def test_contraction_on_a_quantized_workspace(wf, m):
    """Quantize once, contract later: `prefill_quantize` + `bitlinear_batched(workspace=, quantized=True)` equals the
    one-call form bit for bit; one quantization serves several projections of the same tokens (q/k/v like); and a
    chain of stacks launched as independent of one another (each with its own workspace, the first one unmarked)
    gives every stack's one-call result."""
    g = torch.Generator(device=DEV).manual_seed(77 + m)
    k = 1024

    def stack(layers, n):
        codes = torch.empty(layers, n, k // 4, dtype=torch.uint8, device=DEV)
        scales = torch.empty(layers, 2, device=DEV)
        for i in range(layers):
            c, s = wf.pack_ternary(torch.randn(n, k, generator=g, device=DEV) * 0.02)
            codes[i].copy_(c)
            scales[i].copy_(s)
        return codes, scales

    layers = 3
    x = torch.randn(layers, m, k, generator=g, device=DEV).bfloat16()
    projs = [stack(layers, n) for n in (384, 128, 256)]
    want = [wf.bitlinear_batched(x, c, s, out_dtype=torch.float32, want_acc=True) for c, s in projs]
    ws = wf.prefill_workspace(layers * m, k, DEV)
    wf.prefill_quantize(x, ws)
    for (c, s), (y0, a0) in zip(projs, want):
        y, a = wf.bitlinear_batched(torch.zeros_like(x), c, s, out_dtype=torch.float32, want_acc=True, workspace=ws, quantized=True)
        assert torch.equal(a, a0) and torch.equal(y, y0)  # x itself is not read again

    # a chain of independent stacks, as a step over many layer stacks issues them
    chain = []
    for i in range(5):
        xi = torch.randn(layers + i, m, k, generator=g, device=DEV).bfloat16()
        ci, si = stack(layers + i, 640 if i % 2 else 256)
        chain.append((xi, ci, si, wf.bitlinear_batched(xi, ci, si), wf.prefill_workspace((layers + i) * m, k, DEV)))
    torch.cuda.synchronize()
    outs = [torch.empty_like(w) for _, _, _, w, _ in chain]
    for xi, _, _, _, wsi in chain:
        wf.prefill_quantize(xi, wsi, independent=True)  # nothing ahead of them touches x or the workspaces
    for j, (xi, ci, si, _, wsi) in enumerate(chain):
        wf.bitlinear_batched(xi, ci, si, out=outs[j], workspace=wsi, quantized=True, independent=j > 0)
    torch.cuda.synchronize()
    for j, (_, _, _, w, _) in enumerate(chain):
        assert torch.equal(outs[j], w), j
    with pytest.raises(ValueError):
        wf.bitlinear_batched(x, *projs[0], quantized=True)
    wf.device_status()


@pytest.mark.parametrize("m", [16, 32, 64, 128])
def test_contraction_forms_on_a_long_stack(wf, m):
    """Every form of the contraction on a stack with some twenty tiles per CTA (30 layers of 6912 x 2560), launched
    several times back to back on one quantized workspace, alternately as independent launches: the persistent
    pipeline (ring slots, issuing threads, accumulator buffers) keeps its bookkeeping over many tiles and from one
    launch into the next.  Three layers are compared with the per-layer kernels bit for bit."""
    g = torch.Generator(device=DEV).manual_seed(900 + m)
    n, k, layers = 6912, 2560, 30
    codes = torch.empty(layers, n, k // 4, dtype=torch.uint8, device=DEV)
    scales = torch.empty(layers, 2, device=DEV)
    for i in range(layers):
        c, s = wf.pack_ternary(torch.randn(n, k, generator=g, device=DEV) * 0.02)
        codes[i].copy_(c)
        scales[i].copy_(s)
    x = torch.randn(layers, m, k, generator=g, device=DEV).bfloat16()
    y = torch.empty(layers, m, n, dtype=torch.bfloat16, device=DEV)
    picks = (0, layers // 2, layers - 1)
    ref = {i: wf.bitlinear(x[i], codes[i], scales[i], path="decode" if m <= 64 else "prefill") for i in picks}
    ws = wf.prefill_workspace(layers * m, k, DEV)
    wf.prefill_quantize(x, ws)
    for rep in range(6):
        wf.bitlinear_batched(x, codes, scales, out=y, workspace=ws, quantized=True, independent=rep % 2 == 1)
    torch.cuda.synchronize()
    wf.device_status()
    for i in picks:
        assert torch.equal(ref[i], y[i]), i
