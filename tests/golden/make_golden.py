"""Generate the golden vectors under tests/golden/ from the reference itself.

Run where a checkout of the reference project is available:

    python tests/golden/make_golden.py --ref <checkout> [--only cases,packers,ggml,model]

(`--ref` defaults to $WF_REFERENCE_ROOT, else a directory `reference` beside the repository.)
It imports the reference's PyTorch BitLinear, quantization helpers and BitNetLlama model, its
inference-side packers, and calls its compiled CPU kernels (oracle/_ref, built by
`make -C oracle REF=<checkout>`), all on the seeded inputs of tests/golden/inputs.py, and
writes one compressed .npz per case plus packers.npz, ggml.npz and model_<act>.npz.  The tests
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
    from oracle.clib import reference_root

    ap = argparse.ArgumentParser()
    ap.add_argument("--ref", default=reference_root())
    ap.add_argument("--only", default="cases,packers,ggml,model")
    args = ap.parse_args()
    ref = args.ref
    if not ref:
        raise SystemExit("no reference checkout: pass --ref or set WF_REFERENCE_ROOT")
    os.environ["WF_REFERENCE_ROOT"] = ref
    only = set(args.only.split(","))
    sys.path.insert(0, os.path.join(ref, "packages/training/src"))
    sys.path.insert(0, os.path.join(ref, "packages/inference/src"))
    torch.set_num_threads(1)  # fixed reduction order for the stored reference outputs
    if "cases" in only:
        cases()
    if "packers" in only:
        packers(ref)
    if "ggml" in only:
        ggml()
    if "model" in only:
        model()


def cases():

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


def packers(ref):
    """Packers of the inference package."""
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
        # the same quantizer on raw (Gaussian) weights: max-abs scale, +-0.5 thresholds, and the apply() of its class
        from wrinklefree_inference.sglang_backend.bitnet_quantization import BitNetLinearMethod

        p6, s6 = quantize_to_bitnet(w)
        pk["qtb_w_msb"] = p6.numpy()
        pk["qtb_w_scale"] = np.float32(s6)
        xq = torch.randn(5, 256, generator=g)
        pk["qtb_x"] = xq.numpy()
        pk["qtb_apply_bf16"] = BitNetLinearMethod().apply(p6, s6, xq, 16, 256).float().numpy()
    except Exception as e:  # pragma: no cover
        print("bitnet_quantization unavailable:", e)
    np.savez_compressed(os.path.join(HERE, "packers.npz"), **pk)
    print("packers", sorted(pk))


def ggml():
    """BitNet.cpp's I2_S routines (ggml-bitnet-mad.cpp) on ternary weights times a scale."""
    from oracle.clib import load_ggml_reference

    gg = load_ggml_reference()
    assert gg is not None, "oracle/_ref/libref_ggml_mad_avx2.so missing"
    rng = np.random.default_rng(41)
    out = {}
    for tag, (n, k, b) in {"a": (24, 256, 3), "b": (16, 4096 + 128, 2)}.items():  # b: more than 32 blocks per row
        t = rng.integers(-1, 2, size=(n, k)).astype(np.int8)
        w = t.astype(np.float32) * np.float32(0.0371)
        w[0, :4] = [5e-7, -5e-7, 0.0371, -0.0371]  # below the 1e-6 dead zone -> code 0
        packed, scale = gg.quantize_i2_s(w)
        q = rng.integers(-127, 128, size=(b, k)).astype(np.int8)
        sums = q.astype(np.int64).sum(1).astype(np.float32)
        scales = (rng.random(b).astype(np.float32) + 0.5) * 30
        out[f"{tag}_w"], out[f"{tag}_packed"], out[f"{tag}_scale"], out[f"{tag}_q"] = w, packed, scale, q
        out[f"{tag}_act_scales"] = scales
        out[f"{tag}_vec_dot"] = np.array([[gg.vec_dot(packed[r], q[i]) for r in range(n)] for i in range(b)], np.float32)
        out[f"{tag}_mul_mat"] = gg.mul_mat(packed, q, sums, scales, float(scale))
    np.savez_compressed(os.path.join(HERE, "ggml.npz"), **out)
    print("ggml", {kk: getattr(v, "shape", v) for kk, v in out.items()})


def model():
    """The reference's BitNetLlama (llama.py:13-159) at the fixture decoder's size, fp32 and bf16, both activations."""
    from wrinklefree.models.config import BitNetConfig
    from wrinklefree.models.llama import BitNetLlama

    c = gi.MODEL_CFG
    ids = gi.model_ids()
    weights = gi.model_weights()
    for act in ("relu2", "silu"):
        cfg = BitNetConfig(vocab_size=c["vocab"], hidden_size=c["hidden"], intermediate_size=c["intermediate"],
                           num_hidden_layers=c["layers"], num_attention_heads=c["n_q"], num_kv_heads=c["n_kv"],
                           head_dim=c["head_dim"], max_position_embeddings=c["max_pos"], rope_theta=c["rope_theta"],
                           hidden_act=act, rms_norm_eps=c["norm_eps"], tie_word_embeddings=False, use_flash_attention=False)
        out = {"input_sha": gi.sha(ids.numpy(), *[weights[k].numpy() for k in sorted(weights)])}
        for tag, dt in (("f32", torch.float32), ("bf16", torch.bfloat16)):
            m = BitNetLlama(cfg)
            missing, unexpected = m.load_state_dict(weights, strict=False)
            assert not unexpected and all("freqs_cis" in k for k in missing), (missing, unexpected)
            for prm in m.parameters():  # parameters only: Module.to() would also cast the complex RoPE table to real
                prm.data = prm.data.to(dt)
            m.eval()
            with torch.no_grad():
                logits = m(ids)["logits"]
            out[f"logits_{tag}"] = logits[:, gi.MODEL_KEEP_FROM:].float().numpy()
        np.savez_compressed(os.path.join(HERE, f"model_{act}.npz"), **out)
        print("model", act, {kk: getattr(v, "shape", v) for kk, v in out.items() if kk != "input_sha"})


if __name__ == "__main__":
    main()
