"""Module surgery that turns a LLaMA-style model into its BitLinear form, with the reference's names and
results (wrinklefree/training/stage1.py:29-214, wrinklefree/models/subln.py:7-97): every q/k/v/gate/up
projection becomes a BitLinear holding the same parameters, and o_proj / down_proj become
``Sequential(SubLN, BitLinear)`` so that the sub-layer norm runs in front of the output projection.
The BitLinear produced here is this package's drop-in, so converted models run their projections on the
CUDA kernels under ``torch.no_grad()``.
"""
from __future__ import annotations

from typing import Iterable, Optional

import torch
import torch.nn as nn

from .bitlinear import BitLinear


class SubLN(nn.Module):
    """RMS normalisation in front of an output projection: x * rsqrt(mean(x^2) + eps) * weight."""

    def __init__(self, hidden_size: int, eps: float = 1e-6, elementwise_affine: bool = True):
        super().__init__()
        self.hidden_size, self.eps, self.elementwise_affine = hidden_size, eps, elementwise_affine
        if elementwise_affine:
            self.weight = nn.Parameter(torch.ones(hidden_size))
        else:
            self.register_parameter("weight", None)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        y = x * torch.rsqrt(x.pow(2).mean(dim=-1, keepdim=True) + self.eps)
        return y if self.weight is None else y * self.weight

    def extra_repr(self) -> str:
        return f"{self.hidden_size}, eps={self.eps}, elementwise_affine={self.elementwise_affine}"


class RMSNorm(SubLN):
    """The same normalisation under the name the layer norms of the model use."""

    def __init__(self, hidden_size: int, eps: float = 1e-6):
        super().__init__(hidden_size, eps, True)


def _as_bitlinear(proj: nn.Module) -> nn.Module:
    """A BitLinear with the parameters of `proj` (a plain nn.Linear); anything else is returned unchanged."""
    if not isinstance(proj, nn.Linear) or isinstance(proj, BitLinear):
        return proj
    new = BitLinear(proj.in_features, proj.out_features, bias=proj.bias is not None)
    new = new.to(device=proj.weight.device, dtype=proj.weight.dtype)
    new.weight.data.copy_(proj.weight.data)
    if proj.bias is not None:
        new.bias.data.copy_(proj.bias.data)
    new.invalidate_packed()
    return new


def _convert_block(module: nn.Module, inputs: Iterable[str], output: str, fallback_width: int, exclude: list) -> None:
    for name in inputs:
        if hasattr(module, name) and name not in exclude:
            setattr(module, name, _as_bitlinear(getattr(module, name)))
    if hasattr(module, output) and output not in exclude:
        proj = getattr(module, output)
        width = proj.in_features if isinstance(proj, nn.Linear) else fallback_width
        norm = SubLN(width)
        if isinstance(proj, nn.Linear):
            norm = norm.to(device=proj.weight.device)
        setattr(module, output, nn.Sequential(norm, _as_bitlinear(proj)))


def convert_attention_layer(attention_module: nn.Module, hidden_size: int, exclude_layers: list) -> None:
    """q/k/v -> BitLinear, o_proj -> Sequential(SubLN, BitLinear) (stage1.py:63-111)."""
    _convert_block(attention_module, ("q_proj", "k_proj", "v_proj"), "o_proj", hidden_size, exclude_layers)


def convert_mlp_layer(mlp_module: nn.Module, hidden_size: int, exclude_layers: list) -> None:
    """gate/up -> BitLinear, down_proj -> Sequential(SubLN, BitLinear) (stage1.py:114-166)."""
    _convert_block(mlp_module, ("gate_proj", "up_proj"), "down_proj", hidden_size, exclude_layers)


def convert_model_to_bitnet(model: nn.Module, hidden_size: int, intermediate_size: int,
                            exclude_layers: Optional[list] = None) -> nn.Module:
    """Stage-1 conversion of a LLaMA-style model (stage1.py:169-214): modules whose name contains "self_attn" /
    "attention" and that own a q_proj are converted as attention blocks, modules named "mlp" / "feed_forward"
    that own a gate_proj as MLP blocks; names containing an excluded string are skipped."""
    exclude = exclude_layers or ["embed_tokens", "lm_head", "embed_positions"]
    for name, module in list(model.named_modules()):
        if any(e in name for e in exclude):
            continue
        if ("self_attn" in name or "attention" in name) and hasattr(module, "q_proj"):
            convert_attention_layer(module, hidden_size, exclude)
        if ("mlp" in name or "feed_forward" in name) and hasattr(module, "gate_proj"):
            convert_mlp_layer(module, intermediate_size, exclude)
    return model
