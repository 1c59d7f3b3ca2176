"""CPU-side checks: the C-ABI library loads and exports every symbol the header declares,
argument validation answers without a GPU, and the host-side module logic (lambda warm-up,
the straight-through training formula, state_dict compatibility) behaves as the reference's."""
import ctypes
import os
import re

import numpy as np
import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def header_symbols():
    text = open(os.path.join(ROOT, "include", "wf_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(wf_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol(wf):
    lib = ctypes.CDLL(wf._lib.LIB_PATH)
    names = header_symbols()
    assert len(names) >= 12
    for n in names:
        assert hasattr(lib, n), f"{n} declared in include/wf_b200.h but not exported"
    assert sorted(wf._lib.exported_symbols()) == names  # the Python binding covers the whole header


def test_argument_errors_need_no_gpu(wf):
    lib = wf._lib.lib()
    assert lib.wf_version() >= 100
    rc = lib.wf_pack_ternary(None, 0, 4, 64, 64, 0, 1e-5, None, None, None, 0, None)
    assert rc == 1 and b"null pointer" in lib.wf_last_error()
    assert lib.wf_pack_scratch_bytes(1536, 576) >= 8
    assert lib.wf_prefill_workspace_bytes(512, 2560) >= 512 * 2560 + 512 * 4
    buf = (ctypes.c_char * 4096)()
    p = ctypes.addressof(buf)
    p = (p + 255) // 256 * 256
    # K not a multiple of 64 is rejected before anything is launched
    rc = lib.wf_bitlinear_decode(p, 2, 48, None, p, 0, None, 1.0, None, 0, p, 0, 16, None, 1, 16, 48, 1e-5, 0, None)
    assert rc == 1 and b"multiple of 64" in lib.wf_last_error()
    rc = lib.wf_bitlinear_decode(p, 2, 64, None, p, 1, None, 1.0, None, 0, p, 0, 16, None, 1, 16, 64, 1e-5, 0, None)
    assert rc == 1 and b"128" in lib.wf_last_error()


def test_no_cpu_fallback(wf):
    if torch.cuda.is_available():
        pytest.skip("checks the behaviour of a machine without a GPU")
    assert not wf.check_kernel_available()
    with pytest.raises(RuntimeError):
        wf.pack_ternary(torch.zeros(4, 64))
    layer = wf.BitLinear(64, 8)
    with pytest.raises(RuntimeError), torch.no_grad():
        layer(torch.zeros(1, 64))


def test_training_formula_and_lambda(wf):
    torch.manual_seed(0)
    layer = wf.BitLinear(64, 16, bias=True)
    x = torch.randn(3, 64, requires_grad=True)
    # lambda = 1: forward == F.linear(aq(x), wq(W)) (test_paper_verification.py:365-377)
    y = layer(x)
    want = torch.nn.functional.linear(layer.activation_quant(x), layer.weight_quant(layer.weight), layer.bias)
    assert torch.allclose(y, want, atol=1e-5)
    y.sum().backward()
    assert x.grad is not None and layer.weight.grad is not None  # straight-through gradients
    # lambda = 0: plain linear (test_paper_verification.py:353-363)
    warm = wf.LambdaWarmup(warmup_steps=10)
    wf.set_global_lambda_warmup(warm)
    try:
        assert wf.get_current_lambda() == 0.0
        assert torch.allclose(layer(x), torch.nn.functional.linear(x, layer.weight, layer.bias), atol=1e-6)
        for _ in range(5):
            warm.step()
        assert wf.get_current_lambda() == pytest.approx(0.5)
        for _ in range(5):
            warm.step()
        assert warm.is_warmup_complete() and wf.get_current_lambda() == 1.0
        st = warm.state_dict()
        w2 = wf.LambdaWarmup(warmup_steps=3)
        w2.load_state_dict(st)
        assert w2.lambda_val == 1.0 and w2.warmup_steps == 10
    finally:
        wf.set_global_lambda_warmup(None)
    # quantizer formulas (test_paper_verification.py:24-48, 87-110)
    w = torch.randn(16, 64)
    s = w.abs().mean()
    assert torch.allclose(layer.weight_quant(w), (w / s).round().clamp(-1, 1) * s, atol=1e-6)
    aq = layer.activation_quant(x.detach())
    ints = aq * (127.0 / x.detach().abs().max(dim=-1, keepdim=True).values)
    assert torch.allclose(ints, ints.round(), atol=1e-3) and ints.abs().max() <= 128


def test_state_dict_and_conversion(wf):
    lin = torch.nn.Sequential(torch.nn.Linear(64, 32, bias=True), torch.nn.ReLU(), torch.nn.Linear(32, 8, bias=False))
    ref_sd = {k: v.clone() for k, v in lin.state_dict().items()}
    wf.convert_linear_to_bitlinear(lin)
    assert isinstance(lin[0], wf.BitLinear) and isinstance(lin[2], wf.BitLinear)
    assert set(lin.state_dict()) == set(ref_sd)  # weight / bias only: nn.Linear checkpoints load unchanged
    for k, v in ref_sd.items():
        assert torch.equal(lin.state_dict()[k], v)
    other = wf.BitLinear(64, 32, bias=True)
    other.load_state_dict({"weight": ref_sd["0.weight"], "bias": ref_sd["0.bias"]})
    x = torch.randn(2, 64)
    na = wf.BitLinearNoActivationQuant(64, 32)
    na.weight.data.copy_(ref_sd["0.weight"])
    assert torch.allclose(na(x), torch.nn.functional.linear(x, na.weight_quant(na.weight)), atol=1e-6)


def test_linear_method_shapes_on_cpu(wf):
    m = wf.BitNetLinearMethod(wf.BitNetConfig.from_config({"block_size": 128}))
    layer = torch.nn.Module()
    m.create_weights(layer, 256, [64, 64], 256, 128, torch.bfloat16, weight_loader="loader")
    assert layer.qweight.shape == (128, 64) and layer.qweight.dtype == torch.uint8
    assert layer.qweight.input_dim == 1 and layer.qweight.output_dim == 0 and layer.qweight.packed_dim == 1
    assert layer.qweight.weight_loader == "loader" and layer.scale.shape == (1,)
    assert wf.BitNetConfig.get_name() == "bitnet"
    with pytest.raises(RuntimeError):
        if torch.cuda.is_available():
            raise RuntimeError("skip")
        m.apply(layer, torch.zeros(1, 256))
