"""GPU tests of the reference-facing boundary beyond the BitLinear module: the first-party linear methods on the
bytes their own packers emit, the max-abs quantizers against the reference packers' goldens, BitNet.cpp's I2_S
routines (goldens made by its own compiled source), the torch operators, and the contraction at the full sizes of
the prefill configuration against the CPU oracle."""
import os

import numpy as np
import pytest
import torch

import inputs as gi
from oracle import bitlinear_oracle as O

pytestmark = pytest.mark.gpu
GOLD = os.path.join(os.path.dirname(__file__), "golden")
DEV = "cuda:0"


def norm_err(a, b):
    return float(np.abs(a - b).max() / max(np.abs(b).max(), 1e-30))


# ---------------------------------------------------------------- first-party classes on their packers' bytes
def test_first_party_methods_take_their_packers_layouts(wf, oracle_c):
    z = np.load(os.path.join(GOLD, "packers.npz"))
    L = wf._lib
    t = z["ternary"]  # [16, 256] in {-1, 0, 1}
    n, k = t.shape
    g = torch.Generator().manual_seed(5)
    x = torch.randn(6, k, generator=g)
    q, s = oracle_c.act_quant(x.bfloat16().float().numpy(), 1)
    acc = oracle_c.int_gemm(q, t)
    # quantize_to_bitnet's MSB-first bytes through the class that sits beside it (bitnet_quantization.py:366-409)
    msb = torch.from_numpy(z["quantize_to_bitnet_msb"]).to(DEV)
    meth = wf.PackedBitNetLinearMethod()
    y = meth.apply(msb, float(z["quantize_to_bitnet_scale"]), x.to(DEV), n, k)
    want = torch.from_numpy(oracle_c.rescale(acc, s, float(z["quantize_to_bitnet_scale"]))).bfloat16()
    assert y.dtype == torch.bfloat16 and torch.equal(y.cpu(), want)
    assert len(meth._cache) == 1
    meth.apply(msb, 1.0, x.to(DEV), n, k)
    assert len(meth._cache) == 1  # converted once
    meth.clear_cache()
    assert not meth._cache
    # feeding it another layout's bytes with the default must NOT give the same numbers (the old silent mismatch)
    i2s = torch.from_numpy(z["sglkernel_simd"]).to(DEV)
    assert not torch.equal(meth.apply(i2s, 1.0, x.to(DEV), n, k).cpu(), want)
    assert torch.equal(wf.PackedBitNetLinearMethod(layout=L.LAYOUT_I2S).apply(i2s, 1.0, x.to(DEV), n, k).cpu(), want)
    # pack_ternary_weights' LSB-first bytes through BitNetLinearNative (bitnet_patch.py:28-112)
    lsb = torch.from_numpy(z["patch_seq_lsb"]).to(DEV)
    assert np.array_equal(z["patch_seq_lsb"], z["native_seq_lsb"])
    nat = wf.BitNetLinearNative(k, n, lsb, torch.tensor(1.0, device=DEV))
    yn = nat(x.bfloat16().to(DEV))
    assert torch.equal(yn.cpu(), want)
    assert torch.equal(nat.packed_weight, lsb)  # the caller's bytes stay in the buffer
    # its per-tensor arithmetic (one activation scale for the batch), as that class composes it
    natt = wf.BitNetLinearNative(k, n, lsb, torch.tensor(1.0, device=DEV), act_quant="per_tensor")
    mx = np.abs(x.numpy()).max()
    qt = np.clip(np.rint(x.numpy() * (np.float32(127.0) / mx)), -127, 127).astype(np.int8)
    want_t = oracle_c.int_gemm(qt, t).astype(np.float32) * np.float32(mx / np.float32(127.0))
    assert norm_err(natt(x.to(DEV)).cpu().numpy(), want_t) < 1e-6
    # the GPU twins of the packers emit the reference packers' bytes
    p, sc = wf.pack_ternary_weights(torch.from_numpy(t).float().to(DEV))
    assert np.array_equal(p.cpu().numpy(), z["patch_seq_lsb"]) and float(sc) == 1.0
    p2, sc2 = wf.quantize_to_bitnet(torch.from_numpy(t).float().to(DEV))
    assert np.array_equal(p2.cpu().numpy(), z["quantize_to_bitnet_msb"]) and float(sc2) == float(z["quantize_to_bitnet_scale"])
    deq = wf.dequantize_bitnet(p2, sc2, n, k)
    assert np.array_equal(deq.cpu().numpy(), z["dequantize_bitnet"])


def test_quantize_to_bitnet_on_raw_weights(wf):
    """Max-abs scale with thresholds at half of it, on Gaussian weights: bytes and scale equal the reference's, and
    its apply() (bf16 matmul on dequantized weights, no activation quantization) is met within W2A8 tolerance."""
    z = np.load(os.path.join(GOLD, "packers.npz"))
    w = torch.from_numpy(z["w"]).to(DEV)
    p, s = wf.quantize_to_bitnet(w)
    assert np.array_equal(p.cpu().numpy(), z["qtb_w_msb"])
    assert float(s) == float(z["qtb_w_scale"])
    for dt in (torch.bfloat16, torch.float16):  # same codes from low-precision storage of the same values
        p_l, s_l = wf.quantize_to_bitnet(w.to(dt).float())
        p_d, s_d = wf.quantize_to_bitnet(w.to(dt))
        assert torch.equal(p_l, p_d) and torch.equal(s_l, s_d)
    y = wf.PackedBitNetLinearMethod().apply(p, s, torch.from_numpy(z["qtb_x"]).to(DEV), 16, 256)
    assert norm_err(y.float().cpu().numpy(), z["qtb_apply_bf16"]) < 2e-2
    # every row-major destination holds the same codes
    L = wf._lib
    t = wf.unpack_codes(p, 16, 256, L.LAYOUT_SEQ_MSB)
    for lay in (L.LAYOUT_WF16, L.LAYOUT_I2S, L.LAYOUT_SEQ_LSB):
        pl, _ = wf.quantize_maxabs(w, "half", lay)
        assert torch.equal(wf.unpack_codes(pl, 16, 256, lay), t)
        assert torch.equal(wf.repack(p, L.LAYOUT_SEQ_MSB, 16, 256, lay), pl)
    z0, s0 = wf.quantize_to_bitnet(torch.zeros(4, 128, device=DEV))
    assert float(s0) == 1.0 and (wf.unpack_codes(z0, 4, 128, L.LAYOUT_SEQ_MSB) == 0).all()


@pytest.mark.parametrize("tag", ["a", "b"])
def test_bitnet_cpp_i2s_routines(wf, tag):
    """quantize_i2_s and ggml_vec_dot_i2_i8_s (ggml-bitnet-mad.cpp:46-92, 94-): packed bytes and scale identical;
    the raw dot product equals acc + sum(q); the glue arithmetic (ggml.c:12491-12493) within 2 ulp of fp32."""
    z = np.load(os.path.join(GOLD, "ggml.npz"))
    L = wf._lib
    w, q = z[f"{tag}_w"], z[f"{tag}_q"]
    n, k = w.shape
    packed, scale = wf.quantize_maxabs(torch.from_numpy(w).to(DEV), "sign", L.LAYOUT_I2S)
    assert np.array_equal(packed.cpu().numpy(), z[f"{tag}_packed"])
    assert float(scale) == float(z[f"{tag}_scale"])
    qd = torch.from_numpy(q).to(DEV)
    xs = torch.from_numpy(z[f"{tag}_act_scales"]).to(DEV)
    y, acc = wf.bitlinear(qd, packed, scale, layout=L.LAYOUT_I2S, x_scale=xs, want_acc=True)
    raw = acc.cpu().numpy().astype(np.int64) + q.astype(np.int64).sum(1, keepdims=True)
    assert np.array_equal(raw.astype(np.float32), z[f"{tag}_vec_dot"])
    assert np.allclose(y.cpu().numpy(), z[f"{tag}_mul_mat"], rtol=3e-7, atol=0)


def test_torch_operators_on_the_gpu(wf):
    z = np.load(os.path.join(GOLD, "k512.npz"))
    x, w = gi.make_inputs("k512")
    packed = torch.from_numpy(O.pack_i2s(z["codes"])).to(DEV)
    q, s = torch.ops.wf_b200.bitnet_quantize_activations(x.to(DEV))
    assert np.array_equal(q.cpu().numpy(), z["i2s_q_tensor"]) and float(s) == float(z["i2s_act_scale"])
    out = torch.ops.wf_b200.bitnet_gemm(packed, q, float(z["w_scale_torch"]))
    assert np.array_equal(out.cpu().numpy(), z["i2s_gemm"])
    assert np.array_equal(torch.ops.wf_b200.bitnet_gemv(packed, q[0], float(z["w_scale_torch"])).cpu().numpy(), z["i2s_gemv_row0"])
    codes, scale = torch.ops.wf_b200.pack_ternary(w.to(DEV), 0, 1e-5)
    y = torch.ops.wf_b200.bitlinear(x.to(DEV), codes, scale, None, wf._lib.LAYOUT_WF16, 1e-5)
    assert norm_err(y.cpu().numpy(), z["y_f32"]) < 1e-5
    qq, ss = torch.ops.wf_b200.act_quant_i8(x.to(DEV), 1e-5)
    assert np.array_equal(qq.cpu().numpy(), z["q_f32"]) and np.array_equal(ss.cpu().numpy(), z["act_scale_f32"])


# ---------------------------------------------------------------- the prefill configuration at full size
@pytest.mark.parametrize("n,k", [(2560, 2560), (6912, 2560), (2560, 6912)])
@pytest.mark.parametrize("m,form", [(512, "auto"), (2048, "pair"), (2048, "single"), (8192, "pair"), (8192, "single")])
def test_prefill_full_size_against_oracle(wf, oracle_c, n, k, m, form):
    """int8 x ternary GEMM on the tensor cores at the benchmark's shapes: a strided slice of the int32 accumulators
    (every 16th token x every 8th weight row, offsets varied so that every tile position is met) and of the bf16
    outputs against the CPU oracle, bit for bit; row-sum and column-sum checksums over the whole result.  Both tile
    forms of the contraction (one SM per 128 x 128 tile, two SMs per 256 x 192 tile) at the large token counts."""
    g = torch.Generator().manual_seed(n + 3 * k + m)
    w = torch.randn(n, k, generator=g) * 0.02
    x = gi.with_outliers(torch.randn(m, k, generator=g), seed=m + 1).bfloat16()
    codes, scale = wf.pack_ternary(w.to(DEV))
    y, acc = wf.bitlinear(x.to(DEV), codes, scale, want_acc=True, path="prefill", prefill_form=form)
    assert y.dtype == torch.bfloat16
    t_all = wf.unpack_codes(codes, n, k)
    s_w = O.absmean_scale(w.numpy())  # one scale for the whole matrix
    assert float(scale[0]) == float(s_w)
    assert np.array_equal(t_all.cpu().numpy()[::max(1, n // 32)], oracle_c.ternarize(w.numpy()[::max(1, n // 32)], s_w))
    q, s = oracle_c.act_quant(x.float().numpy(), 1)
    toks = np.arange(m)[(np.arange(m) % 16) == (np.arange(m) // 16) % 16]     # one token of every 16, at a moving offset
    rows = np.arange(n)[(np.arange(n) % 8) == (np.arange(n) // 8) % 8]        # one row of every 8, at a moving offset
    t_rows = t_all.cpu().numpy()[rows]
    acc_o = oracle_c.int_gemm(q[toks], t_rows)
    ti, ri = torch.from_numpy(toks).to(DEV), torch.from_numpy(rows).to(DEV)
    assert np.array_equal(acc[ti][:, ri].cpu().numpy(), acc_o)
    y_o = torch.from_numpy(oracle_c.rescale(acc_o, s[toks], float(s_w))).bfloat16()
    assert torch.equal(y[ti][:, ri].cpu(), y_o)
    # checksums over every element: sum_n acc[m, n] = q[m] . sum_n t[n]  and  sum_m acc[m, n] = (sum_m q[m]) . t[n]
    # (fp64 holds these integers exactly: |sums| < 2^53)
    qd = torch.from_numpy(q).to(DEV).double()
    t64 = t_all.double()
    assert torch.equal(acc.double().sum(1), qd @ t64.sum(0))
    assert torch.equal(acc.double().sum(0), t64 @ qd.sum(0))
    # the whole output against the accumulators it was made from (same fp32 operation order on the GPU)
    inv = (1.0 / torch.from_numpy(s).to(DEV)).unsqueeze(1)
    assert torch.equal(y, ((acc.float() * inv) * scale[0]).bfloat16())
    wf.device_status()


def test_weight_only_variant_on_the_bf16_kernel(wf):
    """BitLinearNoActivationQuant at inference: this library's bf16 kernel on the cached quantized weight against the
    reference's formula evaluated by torch (same bf16 operands; the sums differ in order only), the cache follows the weight."""
    torch.manual_seed(3)
    layer = wf.BitLinearNoActivationQuant(576, 200, bias=True).to(DEV)
    x = torch.randn(5, 7, 576, device=DEV).bfloat16()
    with torch.no_grad():
        y = layer(x)
        w = layer.weight.to(torch.bfloat16)
        ref = torch.nn.functional.linear(x.float(), layer.weight_quant(w).float(), layer.bias.float())
    assert y.shape == (5, 7, 200) and y.dtype == torch.bfloat16
    assert float((y.float() - ref).abs().max() / ref.abs().max()) < 1e-2
    with torch.no_grad():
        layer.weight.mul_(-1.0)  # an in-place update is seen through the version counter
        y2 = layer(x)
    ref2 = torch.nn.functional.linear(x.float(), layer.weight_quant(layer.weight.to(torch.bfloat16)).float(), layer.bias.float())
    assert float((y2.float() - ref2).abs().max() / ref2.abs().max()) < 1e-2
    # with a gradient needed the torch formula runs and gradients flow to the weight
    xg = x.clone().requires_grad_(True)
    layer(xg).float().sum().backward()
    assert layer.weight.grad is not None and xg.grad is not None
