"""Drop-in replacement of the reference's BitLinear module
(wrinklefree/models/bitlinear.py:12-192): same class names, constructor,
methods, parameters and state_dict.

At lambda == 1 a CUDA input runs on the packed weights through the C ABI: the
weight is absmean-ternarized and packed once per weight version and input dtype
(an optimizer step changes the version, so the next forward re-packs), and
every forward is a quantize-and-contract kernel.  With gradients enabled the
same forward is wrapped in a straight-through autograd function whose backward
uses the ternary codes and the saved int8 activations.  Only while the lambda
warm-up is active (0 <= lambda < 1 mixes float and quantized operands) and for
gradients on a machine without a GPU does the module evaluate the reference's
formula with torch operators.
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.nn as nn
import torch.nn.functional as F

from . import ops
from .lambda_warmup import get_current_lambda


class _PackedSTE(torch.autograd.Function):
    """Training step of a BitLinear at lambda = 1 on the packed weights (straight-through estimator).

    Forward: per-token int8 quantization + exact integer contraction with the cached ternary codes + fp32 rescale, i.e.
    the value of ``F.linear(activation_quant(x), weight_quant(w), bias)`` without re-ternarizing the latent weight or
    running a float GEMM over integer-valued operands (wrinklefree/models/bitlinear.py:99-113).
    Backward: the gradients autograd derives from the reference's ``v + (quant(v) - v).detach()`` form:
    dX = dY @ weight_quant(w)  (the ternary codes times their scale, unpacked on the GPU for this one product),
    dW = dY^T @ activation_quant(x)  (rebuilt from the saved int8 codes and per-token scales, 1 byte per element saved
    instead of the activation itself), dbias = sum(dY)."""

    @staticmethod
    def forward(ctx, x, weight, bias, layer):
        codes, scale = layer.packed_weight(x.dtype)
        k = x.shape[-1]
        q, s = ops.act_quant_i8(x.reshape(-1, k), eps=layer.eps)
        y = ops.bitlinear(q, codes, scale, bias=bias, x_scale=s, out_dtype=x.dtype)
        ctx.save_for_backward(q, s, codes, scale)
        ctx.in_shape, ctx.x_dtype, ctx.w_dtype = x.shape, x.dtype, weight.dtype
        ctx.has_bias = bias is not None
        return y.reshape(*x.shape[:-1], weight.shape[0])

    @staticmethod
    def backward(ctx, dy):
        q, s, codes, scale = ctx.saved_tensors
        n, k = codes.shape[0], codes.shape[1] * 4
        dy2 = dy.reshape(-1, n)
        dx = dw = db = None
        if ctx.needs_input_grad[0]:
            w_q = ops.unpack_codes(codes, n, k).to(dy2.dtype) * scale[0].to(dy2.dtype)
            dx = (dy2 @ w_q).reshape(ctx.in_shape)
        if ctx.needs_input_grad[1]:
            x_q = q.to(ctx.x_dtype) / s.to(ctx.x_dtype).unsqueeze(1)  # the values activation_quant(x) holds
            dw = (dy2.t() @ x_q.to(dy2.dtype)).to(ctx.w_dtype)
        if ctx.has_bias and ctx.needs_input_grad[2]:
            db = dy2.sum(0)
        return dx, dw, db, None


class BitLinear(nn.Linear):
    """1.58-bit weights (absmean ternary) x 8-bit per-token activations."""

    def __init__(self, in_features: int, out_features: int, bias: bool = False, eps: float = 1e-5):
        super().__init__(in_features, out_features, bias=bias)
        self.eps = eps
        self._packed = {}  # x dtype -> (weight version, data_ptr, codes, scale)

    # ---- the reference's two quantizers, as differentiable-free torch formulas ----
    def weight_quant(self, w: torch.Tensor) -> torch.Tensor:
        scale = 1.0 / w.abs().mean().clamp(min=self.eps)
        return (w * scale).round().clamp(-1, 1) / scale

    def activation_quant(self, x: torch.Tensor) -> torch.Tensor:
        scale = 127.0 / x.abs().max(dim=-1, keepdim=True).values.clamp(min=self.eps)
        return (x * scale).round().clamp(-128, 127) / scale

    # ---- packed weights ----
    def packed_weight(self, dtype: torch.dtype = torch.float32):
        """(codes uint8 [N, K/4], scale float32 [2]) for inputs of `dtype`, rebuilt when the
        weight tensor changes (in-place update or reassignment)."""
        key = (self.weight._version, self.weight.data_ptr(), self.weight.device)
        hit = self._packed.get(dtype)
        if hit is None or hit[0] != key:
            codes, scale = ops.pack_ternary(self.weight.detach(), mode=dtype, eps=self.eps)
            hit = (key, codes, scale)
            self._packed[dtype] = hit
        return hit[1], hit[2]

    def invalidate_packed(self) -> None:
        """Drops the packed copies.  In-place updates through autograd-visible operators are noticed by themselves
        (the weight's version counter is part of the cache key); writes through `.data` (weight loaders) are not:
        call this after them.  `load_state_dict` calls it."""
        self._packed.clear()

    def _load_from_state_dict(self, *args, **kwargs):
        super()._load_from_state_dict(*args, **kwargs)
        self.invalidate_packed()

    def _needs_grad(self, x: torch.Tensor) -> bool:
        return torch.is_grad_enabled() and (x.requires_grad or self.weight.requires_grad
                                            or (self.bias is not None and self.bias.requires_grad))

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        lam = get_current_lambda()
        needs_grad = self._needs_grad(x)
        if lam == 1.0 and (x.is_cuda or not needs_grad):
            if not x.is_cuda:
                raise RuntimeError("BitLinear inference runs on the CUDA kernels only; got a CPU tensor "
                                   "(there is no CPU fallback)")
            if x.dtype not in (torch.float32, torch.bfloat16, torch.float16):
                raise TypeError(f"BitLinear: unsupported input dtype {x.dtype}")
            if needs_grad:  # training at full quantization: packed forward, straight-through backward
                return _PackedSTE.apply(x, self.weight, self.bias, self)
            codes, scale = self.packed_weight(x.dtype)
            return ops.bitlinear(x, codes, scale, bias=self.bias, out_dtype=x.dtype, eps=self.eps)
        # the reference's formula with torch operators: lambda warm-up (0 < lambda < 1 mixes float and quantized
        # operands, which is no single packed product), and gradients on a machine without a GPU
        w = self.weight.to(x.dtype)
        w_quant = w + lam * (self.weight_quant(w) - w).detach()
        x_quant = x + lam * (self.activation_quant(x) - x).detach()
        bias = self.bias.to(x.dtype) if self.bias is not None else None
        return F.linear(x_quant, w_quant, bias)


class BitLinearNoActivationQuant(nn.Linear):
    """Weight-only variant (wrinklefree/models/bitlinear.py:116-151): ternary weights, activations as they are.
    Inference on bf16 CUDA tensors at lambda == 1 runs this library's bf16 tensor-core kernel on the quantized weight,
    which is computed once by the reference's own formula (in bf16, like the reference's forward) and kept until the
    weight changes; everything else evaluates the formula with torch operators."""

    def __init__(self, in_features: int, out_features: int, bias: bool = False, eps: float = 1e-5):
        super().__init__(in_features, out_features, bias=bias)
        self.eps = eps
        self._wq = None  # (key, quantized weight in bf16)

    def weight_quant(self, w: torch.Tensor) -> torch.Tensor:
        scale = 1.0 / w.abs().mean().clamp(min=self.eps)
        return (w * scale).round().clamp(-1, 1) / scale

    def invalidate_packed(self) -> None:
        """Drops the cached quantized weight (after writes through `.data`; `load_state_dict` calls it)."""
        self._wq = None

    def _load_from_state_dict(self, *args, **kwargs):
        super()._load_from_state_dict(*args, **kwargs)
        self.invalidate_packed()

    def quantized_weight(self) -> torch.Tensor:
        key = (self.weight._version, self.weight.data_ptr(), self.weight.device)
        if self._wq is None or self._wq[0] != key:
            with torch.no_grad():
                self._wq = (key, self.weight_quant(self.weight.detach().to(torch.bfloat16)).contiguous())
        return self._wq[1]

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        lam = get_current_lambda()
        needs_grad = torch.is_grad_enabled() and (x.requires_grad or self.weight.requires_grad
                                                  or (self.bias is not None and self.bias.requires_grad))
        if (lam == 1.0 and not needs_grad and x.is_cuda and x.dtype == torch.bfloat16 and self.in_features % 8 == 0):
            y = ops.linear_bf16(x, self.quantized_weight())
            return y if self.bias is None else y + self.bias.to(x.dtype)
        w = self.weight.to(x.dtype)
        w_quant = w + lam * (self.weight_quant(w) - w).detach()
        bias = self.bias.to(x.dtype) if self.bias is not None else None
        return F.linear(x, w_quant, bias)


def convert_linear_to_bitlinear(module: nn.Module, exclude_names: Optional[list] = None) -> nn.Module:
    """Replace every nn.Linear below `module` by a BitLinear holding the same parameters
    (wrinklefree/models/bitlinear.py:154-192)."""
    exclude_names = exclude_names or []
    for name, child in module.named_children():
        if name in exclude_names:
            continue
        if isinstance(child, nn.Linear) and not isinstance(child, BitLinear):
            new = BitLinear(child.in_features, child.out_features, bias=child.bias is not None)
            new = new.to(device=child.weight.device, dtype=child.weight.dtype)
            new.weight.data.copy_(child.weight.data)
            if child.bias is not None:
                new.bias.data.copy_(child.bias.data)
            new.invalidate_packed()
            setattr(module, name, new)
        else:
            convert_linear_to_bitlinear(child, exclude_names)
    return module
