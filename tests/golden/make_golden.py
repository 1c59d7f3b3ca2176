"""Generate the golden vectors under tests/golden/ from the reference itself.

Run where the reference checkout is mounted (default /root/reference):

    python tests/golden/make_golden.py [--ref /root/reference]

It imports the reference's PyTorch BitLinear and quantization helpers, its
inference-side packers, and calls its compiled CPU kernel (oracle/_ref, built by
`make -C oracle`), all on the seeded inputs of tests/golden/inputs.py, and
writes one compressed .npz per case plus packers.npz and kat.npz.  The tests
never need the reference: they read these files.
"""
from __future__ import annotations

import argparse
import importlib.util
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)
sys.path.insert(0, HERE)

import inputs as gi  # noqa: E402


def _load_file(path, name):
    spec = importlib.util.spec_from_file_location(name, path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--ref", default="/root/reference")
    args = ap.parse_args()
    ref = args.ref
    sys.path.insert(0, os.path.join(ref, "packages/training/src"))
    sys.path.insert(0, os.path.join(ref, "packages/inference/src"))

    from wrinklefree.models.bitlinear import BitLinear
    from wrinklefree.quantization.activation_quant import activation_quantization_per_token
    from wrinklefree.quantization.weight_quant import (
        compute_weight_scale,
        ternary_weight_quantization,
        ternary_weight_quantization_no_scale,
    )

    from oracle.clib import build, load_reference

    build()
    refk = load_reference()
    assert refk is not None, "oracle/_ref missing"
    torch.set_num_threads(1)  # fixed reduction order for the stored reference outputs

    for name in gi.CASES:
        m, k, n, seed = gi.CASES[name]
        x, w = gi.make_inputs(name)
        out = {"input_sha": gi.sha(x.numpy(), w.numpy())}

        # --- weights: fp32 ternarization (weight_quant.py:35-56)
        codes_f, scale_t = ternary_weight_quantization_no_scale(w)
        out["codes"] = codes_f.to(torch.int8).numpy()
        out["w_scale_torch"] = scale_t.numpy().astype(np.float32)
        assert float(compute_weight_scale(w)) == float(scale_t)
        # the scaled variant (weight_quant.py:6-32) must carry the same codes
        wq = ternary_weight_quantization(w)
        assert torch.equal(torch.sign(wq).to(torch.int8), codes_f.to(torch.int8))

        layer = BitLinear(k, n, bias=False)
        with torch.no_grad():
            layer.weight.copy_(w)

        for tag, dt in (("f32", torch.float32), ("bf16", torch.bfloat16), ("f16", torch.float16)):
            xd = x.to(dt)
            with torch.no_grad():
                # integers exactly as bitlinear.py:79-82 forms them
                scale = 127.0 / xd.abs().max(dim=-1, keepdim=True).values.clamp(min=layer.eps)
                q = (xd * scale).round().clamp(-128, 127)
                aq = layer.activation_quant(xd)
                assert torch.equal(aq, q / scale)
                assert torch.equal(aq, activation_quantization_per_token(xd))
                out[f"q_{tag}"] = q.to(torch.int8).numpy()
                out[f"act_scale_{tag}"] = scale.float().reshape(-1).numpy()
                # cast-first weight quantization of the forward (bitlinear.py:103-107)
                wl = layer.weight.to(dt)
                wq_l = layer.weight_quant(wl)
                out[f"codes_fwd_{tag}"] = torch.sign(wq_l.float()).to(torch.int8).numpy()
                out[f"dequant_fwd_{tag}"] = np.float32(wq_l.float().abs().max().item())
                y = layer(xd)
                assert y.dtype == dt
                out[f"y_{tag}"] = y.float().numpy()
        # a bias variant, fp32 only (test_bitlinear.py bias case)
        lb = BitLinear(k, n, bias=True)
        g = torch.Generator().manual_seed(seed + 1)
        bias = torch.randn(n, generator=g) * 0.1
        with torch.no_grad():
            lb.weight.copy_(w)
            lb.bias.copy_(bias)
            out["bias"] = bias.numpy()
            out["y_bias_f32"] = lb(x).numpy()

        # --- the inference CPU kernel on I2_S weights (K % 128 == 0 only)
        if name in gi.I2S_CASES:
            from oracle import bitlinear_oracle as O

            packed = O.pack_i2s(out["codes"])
            q_t, s_t = refk.quantize_activations(x.numpy())
            out["i2s_q_tensor"] = q_t
            out["i2s_act_scale"] = np.float32(s_t)
            out["i2s_gemm"] = refk.gemm(packed, q_t.reshape(m, k), float(scale_t))
            out["i2s_gemv_row0"] = refk.gemv(packed, q_t.reshape(m, k)[0], float(scale_t))
        np.savez_compressed(os.path.join(HERE, f"{name}.npz"), **out)
        print(name, {kk: getattr(v, "shape", v) for kk, v in out.items() if kk != "input_sha"})

    # ---------------- packers of the inference package ----------------
    pk = {}
    g = torch.Generator().manual_seed(21)
    w = torch.randn(16, 256, generator=g) * 0.02
    pk["w"] = w.numpy()
    conv = _load_file(os.path.join(ref, "packages/inference/scripts/convert_to_sglkernel.py"), "ref_convert")
    p, s = conv.pack_ternary_sglkernel(w, simd_mode=True)
    pk["sglkernel_simd"] = p.numpy()
    pk["sglkernel_scale"] = np.float32(s)
    p2, _ = conv.pack_ternary_sglkernel(w, simd_mode=False)
    pk["sglkernel_scalar"] = p2.numpy()
    tern = (w / w.abs().mean()).round().clamp(-1, 1)
    pk["ternary"] = tern.to(torch.int8).numpy()
    core = _load_file(os.path.join(ref, "packages/inference/tests/test_bitnet_core.py"), "ref_core")
    p3, _ = core._pack_ternary_weights(tern)
    pk["core_blocked"] = p3.numpy()
    assert torch.equal(core._unpack_i2_to_ternary(p3, 16, 256), tern.float())
    # HF [N/4, K] layout: the reference only ships the unpacker; pin it on random bytes
    hf = torch.randint(0, 256, (4, 256), generator=g, dtype=torch.int32)
    hf = (hf & 0x03) % 3 | (((hf >> 2) & 3) % 3) << 2 | (((hf >> 4) & 3) % 3) << 4 | (((hf >> 6) & 3) % 3) << 6
    hf = hf.to(torch.uint8)
    pk["hf_bytes"] = hf.numpy()
    pk["hf_unpacked"] = core._unpack_ternary_weights(hf).to(torch.int8).numpy()
    try:
        from wrinklefree_inference.kernels import native as ref_native

        pk["native_seq_lsb"] = ref_native.pack_weights(tern.numpy())
        assert (ref_native.unpack_weights(pk["native_seq_lsb"]) == tern.numpy()).all()
        pk["native_from_hf"] = ref_native.repack_hf_weights(hf.numpy())
    except Exception as e:  # pragma: no cover
        print("native.py unavailable:", e)
    try:
        from wrinklefree_inference.kernels.bitnet_patch import pack_ternary_weights

        p4, _ = pack_ternary_weights(tern)
        pk["patch_seq_lsb"] = p4.numpy()
    except Exception as e:  # pragma: no cover
        print("bitnet_patch unavailable:", e)
    try:
        from wrinklefree_inference.sglang_backend.bitnet_quantization import dequantize_bitnet, quantize_to_bitnet

        p5, s5 = quantize_to_bitnet(tern)  # ternary input, max-abs scale 1 -> thresholds +-0.5
        pk["quantize_to_bitnet_msb"] = p5.numpy()
        pk["quantize_to_bitnet_scale"] = np.float32(s5)
        pk["dequantize_bitnet"] = dequantize_bitnet(p5, s5, 16, 256).float().numpy()
    except Exception as e:  # pragma: no cover
        print("bitnet_quantization unavailable:", e)
    np.savez_compressed(os.path.join(HERE, "packers.npz"), **pk)
    print("packers", sorted(pk))


if __name__ == "__main__":
    main()
