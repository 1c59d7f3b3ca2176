"""The reference's PyTorch BitLinear forward, restated with torch operators (CPU baseline and checker).

TEST INFRASTRUCTURE ONLY, like the rest of this directory: the benchmark times it on the host cores as the
"reference PyTorch BitLinear.forward" baseline (the reference package itself is not present where the benchmark
runs), and tests/test_oracle_golden.py pins it to outputs of the reference's own class.

Restated from packages/training/src/wrinklefree/models/bitlinear.py:
  weight_quant      :46-64   scale = 1 / mean|w|.clamp(eps);  (w * scale).round().clamp(-1, 1) / scale
  activation_quant  :66-84   per token scale = 127 / max|x|.clamp(eps);  (x * scale).round().clamp(-128, 127) / scale
  forward           :86-113  weight cast to x.dtype, both operands re-quantized on every call, F.linear in x.dtype
(lambda = 1: the straight-through `x + (q(x) - x).detach()` equals q(x) in value.)
"""
from __future__ import annotations

import torch
import torch.nn.functional as F

EPS = 1e-5


def weight_quant(w: torch.Tensor, eps: float = EPS) -> torch.Tensor:
    scale = 1.0 / w.abs().mean().clamp(min=eps)
    return (w * scale).round().clamp(-1, 1) / scale


def activation_quant(x: torch.Tensor, eps: float = EPS) -> torch.Tensor:
    scale = 127.0 / x.abs().max(dim=-1, keepdim=True).values.clamp(min=eps)
    return (x * scale).round().clamp(-128, 127) / scale


def bitlinear_forward(x: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor = None, eps: float = EPS) -> torch.Tensor:
    """One call of the reference forward at lambda = 1: everything in x.dtype, weights re-ternarized per call."""
    w = weight.to(x.dtype)
    b = bias.to(x.dtype) if bias is not None else None
    return F.linear(activation_quant(x, eps), weight_quant(w, eps), b)
