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


def test_torch_operators_are_registered_with_fake_shapes(wf):
    """torch.ops.wf_b200.* exist with the reference's operator argument lists, and their shape-only
    implementations answer without a GPU (cpu_graph_runner.py:340-354 registers the same for the CPU operators)."""
    from torch._subclasses.fake_tensor import FakeTensorMode

    for name in wf.torch_ops.OPERATORS:
        assert hasattr(torch.ops.wf_b200, name)
    with FakeTensorMode():
        pw = torch.empty(64, 32, dtype=torch.uint8, device="cuda")
        a = torch.empty(5, 128, dtype=torch.int8, device="cuda")
        out = torch.ops.wf_b200.bitnet_gemm(pw, a, 0.5)
        assert out.shape == (5, 64) and out.dtype == torch.float32
        assert torch.ops.wf_b200.bitnet_gemv(pw, a[0], 0.5).shape == (64,)
        q, s = torch.ops.wf_b200.bitnet_quantize_activations(torch.empty(5, 128, device="cuda"))
        assert q.dtype == torch.int8 and q.shape == (5, 128) and s.shape == (1,)
        x = torch.empty(2, 3, 128, dtype=torch.bfloat16, device="cuda")
        y = torch.ops.wf_b200.bitlinear(x, pw, torch.empty(2, device="cuda"), None, 0, 1e-5)
        assert y.shape == (2, 3, 64) and y.dtype == torch.bfloat16
        c, sc = torch.ops.wf_b200.pack_ternary(torch.empty(16, 256, device="cuda"), 0, 1e-5)
        assert c.shape == (16, 64) and c.dtype == torch.uint8 and sc.shape == (2,)


def test_model_conversion_inserts_subln(wf):
    """convert_model_to_bitnet (stage1.py:169-214): q/k/v/gate/up become BitLinear with the same parameters,
    o_proj / down_proj become Sequential(SubLN, BitLinear); excluded names are left alone."""
    nn = torch.nn

    class Attn(nn.Module):
        def __init__(self):
            super().__init__()
            self.q_proj, self.k_proj, self.v_proj = nn.Linear(64, 64, bias=False), nn.Linear(64, 32), nn.Linear(64, 32)
            self.o_proj = nn.Linear(64, 64, bias=False)

    class Mlp(nn.Module):
        def __init__(self):
            super().__init__()
            self.gate_proj, self.up_proj, self.down_proj = nn.Linear(64, 128), nn.Linear(64, 128), nn.Linear(128, 64)

    class Layer(nn.Module):
        def __init__(self):
            super().__init__()
            self.self_attn, self.mlp = Attn(), Mlp()

    class Model(nn.Module):
        def __init__(self):
            super().__init__()
            self.embed_tokens = nn.Embedding(10, 64)
            self.layers = nn.ModuleList([Layer(), Layer()])
            self.lm_head = nn.Linear(64, 10, bias=False)

    m = Model()
    before = {k: v.clone() for k, v in m.state_dict().items()}
    wf.convert_model_to_bitnet(m, hidden_size=64, intermediate_size=128)
    for layer in m.layers:
        for name in ("q_proj", "k_proj", "v_proj"):
            assert isinstance(getattr(layer.self_attn, name), wf.BitLinear)
        assert isinstance(layer.self_attn.o_proj, nn.Sequential) and isinstance(layer.self_attn.o_proj[0], wf.SubLN)
        assert isinstance(layer.self_attn.o_proj[1], wf.BitLinear) and layer.self_attn.o_proj[0].hidden_size == 64
        assert isinstance(layer.mlp.down_proj[0], wf.SubLN) and layer.mlp.down_proj[0].hidden_size == 128
        assert isinstance(layer.mlp.gate_proj, wf.BitLinear) and isinstance(layer.mlp.down_proj[1], wf.BitLinear)
    assert type(m.lm_head) is nn.Linear
    assert torch.equal(m.layers[1].mlp.down_proj[1].weight, before["layers.1.mlp.down_proj.weight"])
    assert torch.equal(m.layers[0].self_attn.k_proj.bias, before["layers.0.self_attn.k_proj.bias"])
    x = torch.randn(3, 128)
    sub = m.layers[0].mlp.down_proj[0]
    assert torch.allclose(sub(x), x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + 1e-6), atol=1e-6)
    assert wf.create_bitnet_config(block_size=128).block_size == 128


def _reference_checkout():
    from oracle.clib import reference_root

    return reference_root()


@pytest.mark.skipif(_reference_checkout() is None, reason="needs a checkout of the reference project")
def test_drop_in_inside_the_reference_tree(wf, monkeypatch):
    """The swap a maintainer makes: the reference's own callers (BitNetFFN, BitNetAttention, the stage-1 converter)
    import `wrinklefree.models.bitlinear`; with that module's classes replaced by the drop-in they build drop-in
    layers, `isinstance` checks hold, and the lambda schedule the reference's trainer installs in ITS module is the
    one the drop-in reads."""
    import importlib
    import sys

    ref = _reference_checkout()
    monkeypatch.syspath_prepend(os.path.join(ref, "packages", "training", "src"))
    for name in [n for n in sys.modules if n == "wrinklefree" or n.startswith("wrinklefree.")]:
        monkeypatch.delitem(sys.modules, name)
    ref_bl = importlib.import_module("wrinklefree.models.bitlinear")
    ref_forward_cls = ref_bl.BitLinear
    for name in ("BitLinear", "BitLinearNoActivationQuant", "convert_linear_to_bitlinear"):
        monkeypatch.setattr(ref_bl, name, getattr(wf, name))
    for name in ("wrinklefree.models.ffn", "wrinklefree.models.attention", "wrinklefree.models"):
        sys.modules.pop(name, None)
    ffn_mod = importlib.import_module("wrinklefree.models.ffn")
    att_mod = importlib.import_module("wrinklefree.models.attention")
    ref_lw = importlib.import_module("wrinklefree.quantization.lambda_warmup")

    torch.manual_seed(1)
    ffn = ffn_mod.BitNetFFN(64, 128, hidden_act="relu2")
    att = att_mod.BitNetAttention(64, 4, 2, 16, max_position_embeddings=16)
    assert isinstance(ffn.gate_proj, wf.BitLinear) and isinstance(att.o_proj, wf.BitLinear)
    # same numbers as the reference's own class on the training formula (gradient enabled -> torch formula on CPU)
    x = torch.randn(2, 5, 64, requires_grad=True)
    twin = ref_forward_cls(64, 128)
    twin.weight.data.copy_(ffn.gate_proj.weight.data)
    assert torch.allclose(ffn.gate_proj(x), twin(x), atol=1e-6)
    y = ffn(x)
    y.sum().backward()
    assert y.shape == (2, 5, 64) and ffn.down_proj.weight.grad is not None
    # the trainer's call (training/stage2.py): the schedule goes into the reference module's global
    warm = ref_lw.LambdaWarmup(warmup_steps=4)
    ref_lw.set_global_lambda_warmup(warm)
    try:
        assert wf.get_current_lambda() == 0.0  # the drop-in sees it
        plain = torch.nn.functional.linear(x, ffn.gate_proj.weight)
        assert torch.allclose(ffn.gate_proj(x), plain, atol=1e-6)  # lambda = 0: no quantization
        warm.step()
        warm.step()
        assert wf.get_current_lambda() == pytest.approx(0.5)
        lam_half = ffn.gate_proj(x)
        assert torch.allclose(lam_half, twin(x), atol=1e-6)  # the reference class mixes with the same lambda
        with torch.no_grad():  # lambda < 1 keeps the drop-in off the packed path even without gradients
            assert torch.allclose(ffn.gate_proj(x.detach()), lam_half.detach(), atol=1e-6)
    finally:
        ref_lw.set_global_lambda_warmup(None)
    assert wf.get_current_lambda() == 1.0
    # and the other direction: a schedule installed through the drop-in's module reaches the reference's global
    wf.set_global_lambda_warmup(wf.LambdaWarmup(warmup_steps=2))
    try:
        assert ref_lw.get_current_lambda() == 0.0
    finally:
        wf.set_global_lambda_warmup(None)
    assert ref_lw.get_global_lambda_warmup() is None


def test_packed_weight_cache_invalidation(wf):
    layer = wf.BitLinear(64, 8)
    layer._packed[torch.float32] = ("stale",)
    layer.load_state_dict({"weight": torch.zeros(8, 64)})
    assert not layer._packed  # loaders write through .data: load_state_dict drops the packed copies
    layer._packed[torch.float32] = ("stale",)
    layer.invalidate_packed()
    assert not layer._packed


def test_flags_match_the_header_and_the_stack_rule(wf):
    """The flag values of the Python binding are those of include/wf_b200.h, wf_prefill_quantize validates its
    arguments without a GPU, and the rule that sends a stack of layers to the contraction is monotonic in the token
    count."""
    text = open(os.path.join(ROOT, "include", "wf_b200.h")).read()
    defs = {k: int(v) for k, v in re.findall(r"#define\s+(WF_FLAG_[A-Z_]+)\s+(\d+)u", text)}
    L = wf._lib
    assert defs["WF_FLAG_PDL"] == L.FLAG_PDL and defs["WF_FLAG_X_READY"] == L.FLAG_X_READY
    assert defs["WF_FLAG_WS_READY"] == L.FLAG_WS_READY
    assert defs["WF_FLAG_PREFILL_PAIR"] == L.FLAG_PREFILL_PAIR and defs["WF_FLAG_PREFILL_SINGLE"] == L.FLAG_PREFILL_SINGLE
    assert len(set(defs.values())) == len(defs)  # distinct bits
    lib = L.lib()
    assert lib.wf_prefill_quantize(None, 2, 64, 4, 64, 1e-5, None, 0, 0, None) == 1
    assert b"wf_prefill_quantize" in lib.wf_last_error()
    for k in (2560, 4096, 6912, 14336):
        uses = [wf.stack_uses_contraction(m, k) for m in range(1, 65)]
        assert uses == sorted(uses) and uses[-1] and not uses[0]  # once on the contraction, always from there on
    assert wf.stack_uses_contraction(4, 6912) and not wf.stack_uses_contraction(4, 2560) and wf.stack_uses_contraction(8, 2560)
