"""Torch operator registration on top of the C ABI: ``torch.ops.wf_b200.*``.

The reference exposes its kernels as torch operators with a schema and a fake-tensor (shape-only) implementation,
so that graph capture and ``torch.compile`` can trace through them
(sgl-kernel/csrc/cpu/torch_extension_cpu.cpp:912-918 for the schemas,
python/sglang/srt/model_executor/cpu_graph_runner.py:340-354 for the fake shapes).  The same three operators are
registered here under the same argument lists, plus the operators of the BitLinear path itself.  Every operator has
a CUDA implementation only (it calls the C ABI through ``ops``); there is no CPU implementation to dispatch to.

    wf_b200::bitnet_gemv(Tensor packed_weights, Tensor activations, float scale) -> Tensor                fp32 [N]
    wf_b200::bitnet_gemm(Tensor packed_weights, Tensor activations, float scale) -> Tensor                fp32 [B, N]
    wf_b200::bitnet_quantize_activations(Tensor input) -> (Tensor, Tensor)                                int8, fp32 [1]
    wf_b200::pack_ternary(Tensor weight, int mode, float eps) -> (Tensor, Tensor)                         u8 [N, K/4], fp32 [2]
    wf_b200::act_quant_i8(Tensor x, float eps) -> (Tensor, Tensor)                                        int8, fp32 [M]
    wf_b200::bitlinear(Tensor x, Tensor codes, Tensor w_scale, Tensor? bias, int layout, float eps) -> Tensor   x.dtype [..., N]
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch

from . import _lib as L
from . import ops

_MODE = {0: torch.float32, 1: torch.bfloat16, 2: torch.float16}  # WF_PACK_* -> arithmetic type


@torch.library.custom_op("wf_b200::bitnet_gemv", mutates_args=(), device_types="cuda")
def bitnet_gemv(packed_weights: torch.Tensor, activations: torch.Tensor, scale: float) -> torch.Tensor:
    return ops.bitnet_gemv(packed_weights, activations, scale)


@bitnet_gemv.register_fake
def _(packed_weights, activations, scale):
    return torch.empty(packed_weights.shape[0], dtype=torch.float32, device=packed_weights.device)


@torch.library.custom_op("wf_b200::bitnet_gemm", mutates_args=(), device_types="cuda")
def bitnet_gemm(packed_weights: torch.Tensor, activations: torch.Tensor, scale: float) -> torch.Tensor:
    return ops.bitnet_gemm(packed_weights, activations, scale)


@bitnet_gemm.register_fake
def _(packed_weights, activations, scale):
    return torch.empty(activations.shape[0], packed_weights.shape[0], dtype=torch.float32, device=packed_weights.device)


@torch.library.custom_op("wf_b200::bitnet_quantize_activations", mutates_args=(), device_types="cuda")
def bitnet_quantize_activations(input: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    return ops.quantize_activations_i8(input)


@bitnet_quantize_activations.register_fake
def _(input):
    return torch.empty_like(input, dtype=torch.int8), torch.empty(1, dtype=torch.float32, device=input.device)


@torch.library.custom_op("wf_b200::pack_ternary", mutates_args=(), device_types="cuda")
def pack_ternary(weight: torch.Tensor, mode: int, eps: float) -> Tuple[torch.Tensor, torch.Tensor]:
    return ops.pack_ternary(weight, mode=_MODE[mode], eps=eps)


@pack_ternary.register_fake
def _(weight, mode, eps):
    n, k = weight.shape
    return (torch.empty(n, k // 4, dtype=torch.uint8, device=weight.device),
            torch.empty(2, dtype=torch.float32, device=weight.device))


@torch.library.custom_op("wf_b200::act_quant_i8", mutates_args=(), device_types="cuda")
def act_quant_i8(x: torch.Tensor, eps: float) -> Tuple[torch.Tensor, torch.Tensor]:
    q, s = ops.act_quant_i8(x, eps=eps)
    return q, s


@act_quant_i8.register_fake
def _(x, eps):
    return torch.empty_like(x, dtype=torch.int8), torch.empty(x.numel() // x.shape[-1], dtype=torch.float32, device=x.device)


@torch.library.custom_op("wf_b200::bitlinear", mutates_args=(), device_types="cuda")
def bitlinear(x: torch.Tensor, codes: torch.Tensor, w_scale: torch.Tensor, bias: Optional[torch.Tensor], layout: int,
              eps: float) -> torch.Tensor:
    return ops.bitlinear(x, codes, w_scale, bias=bias, layout=layout, eps=eps)


@bitlinear.register_fake
def _(x, codes, w_scale, bias, layout, eps):
    dt = torch.float32 if x.dtype == torch.int8 else x.dtype
    return torch.empty(*x.shape[:-1], codes.shape[0], dtype=dt, device=x.device)


OPERATORS = ("bitnet_gemv", "bitnet_gemm", "bitnet_quantize_activations", "pack_ternary", "act_quant_i8", "bitlinear")
WF_LAYOUT_WF16, WF_LAYOUT_I2S = L.LAYOUT_WF16, L.LAYOUT_I2S
