"""The inference side's "ternary linear method", with the reference's signatures.

* ``BitNetConfig`` / ``BitNetLinearMethod``: the SGLang quantization plug-in
  (sglang/srt/layers/quantization/bitnet.py:45-255): ``create_weights``,
  ``process_weights_after_loading``, ``apply(layer, x, bias)``.  SGLang itself is
  not needed to import this module; when it is installed the classes can be
  registered under the name "bitnet" unchanged.
* ``PackedBitNetLinearMethod``: the first-party twin whose ``apply`` takes the
  packed weight explicitly (wrinklefree_inference/sglang_backend/bitnet_quantization.py:366-409).
* ``BitNetLinearNative``: the patched module (wrinklefree_inference/kernels/bitnet_patch.py:28-78).

Weights arrive in the I2_S block layout, as checkpoints of the reference store
them; the kernels consume that layout directly.  No host synchronisation
happens in ``apply`` (the reference calls ``scale.item()`` per call).
"""
from __future__ import annotations

from typing import Any, Dict, List, Optional

import torch
import torch.nn as nn
from torch.nn.parameter import Parameter

from . import _lib as L
from . import ops

BITNET_BLOCK_SIZE = 128
BITS_PER_WEIGHT = 1.58


def _set_weight_attrs(weight: torch.Tensor, attrs: Optional[Dict[str, Any]]):
    if attrs:
        for k, v in attrs.items():
            setattr(weight, k, v)


class BitNetConfig:
    """Quantization config named "bitnet"."""

    def __init__(self, block_size: int = BITNET_BLOCK_SIZE, activation_bits: int = 8, act_quant: str = "per_token"):
        self.block_size = block_size
        self.activation_bits = activation_bits
        self.act_quant = act_quant  # "per_token" (BitLinear semantics) or "per_tensor" (the CPU operator's)

    def __repr__(self) -> str:
        return f"BitNetConfig(block_size={self.block_size}, activation_bits={self.activation_bits})"

    @classmethod
    def get_name(cls) -> str:
        return "bitnet"

    @classmethod
    def get_supported_act_dtypes(cls) -> List[torch.dtype]:
        return [torch.int8, torch.float16, torch.bfloat16, torch.float32]

    @classmethod
    def get_min_capability(cls) -> int:
        return 100  # sm_100 kernels only

    @classmethod
    def get_config_filenames(cls) -> List[str]:
        return []

    @classmethod
    def from_config(cls, config: Dict[str, Any]) -> "BitNetConfig":
        return cls(block_size=config.get("block_size", BITNET_BLOCK_SIZE), activation_bits=config.get("activation_bits", 8))

    def get_quant_method(self, layer: nn.Module, prefix: str = ""):
        return BitNetLinearMethod(self)

    def get_scaled_act_names(self) -> List[str]:
        return []


class BitNetLinearMethod:
    """`LinearMethodBase`-shaped plug-in.  NO FALLBACK: raises when the CUDA library is unusable."""

    def __init__(self, quant_config: Optional[BitNetConfig] = None):
        self.quant_config = quant_config or BitNetConfig()

    def create_weights(self, layer: nn.Module, input_size_per_partition: int, output_partition_sizes: List[int],
                       input_size: int, output_size: int, params_dtype: torch.dtype, **extra_weight_attrs):
        if input_size_per_partition % self.quant_config.block_size != 0:
            raise ValueError(f"BitNet: input_size_per_partition ({input_size_per_partition}) "
                             f"must be divisible by block_size ({self.quant_config.block_size})")
        out_per_partition = sum(output_partition_sizes)
        qweight = Parameter(torch.empty((out_per_partition, input_size_per_partition // 4), dtype=torch.uint8),
                            requires_grad=False)
        _set_weight_attrs(qweight, {"input_dim": 1, "output_dim": 0, "packed_dim": 1, "pack_factor": 4,
                                    "is_bitnet_weight": True})
        _set_weight_attrs(qweight, extra_weight_attrs)
        layer.register_parameter("qweight", qweight)
        scale = Parameter(torch.ones(1, dtype=torch.float32), requires_grad=False)
        _set_weight_attrs(scale, {"is_bitnet_scale": True})
        _set_weight_attrs(scale, extra_weight_attrs)
        layer.register_parameter("scale", scale)

    def process_weights_after_loading(self, layer: nn.Module):
        if layer.qweight.dtype != torch.uint8:
            raise ValueError(f"BitNet: Expected qweight dtype uint8, got {layer.qweight.dtype}. "
                             "Model may not be properly quantized for BitNet.")
        if not layer.qweight.is_contiguous():
            layer.qweight.data = layer.qweight.data.contiguous()

    def apply(self, layer: nn.Module, x: torch.Tensor, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
        """x [tokens, in] -> float32 [tokens, out] (dtype of the operator this replaces)."""
        if not ops.check_kernel_available():
            raise RuntimeError("BitNet apply FAILED: the wf_b200 CUDA library is not usable on this device. "
                               "NO FALLBACK is provided.")
        if self.quant_config.act_quant == "per_tensor":
            q, s = ops.quantize_activations_i8(x)
            out = ops.bitlinear(q, layer.qweight, layer.scale, layout=L.LAYOUT_I2S, out_dtype=torch.float32)
            out = out * s
            return out + bias if bias is not None else out
        return ops.bitlinear(x, layer.qweight, layer.scale, bias=bias, layout=L.LAYOUT_I2S, out_dtype=torch.float32)


class PackedBitNetLinearMethod:
    """First-party signature: apply(packed_weight, scale, x, out_features, in_features, bias)."""

    def __init__(self, compute_dtype: torch.dtype = torch.bfloat16, layout: int = L.LAYOUT_I2S):
        self.compute_dtype = compute_dtype
        self.layout = layout

    def apply(self, packed_weight: torch.Tensor, scale, x: torch.Tensor, out_features: int, in_features: int,
              bias: Optional[torch.Tensor] = None, sparsity_config=None) -> torch.Tensor:
        if sparsity_config is not None and getattr(sparsity_config, "enabled", False):
            raise NotImplementedError("activation sparsity is not part of the CUDA path")
        if packed_weight.shape != (out_features, in_features // 4):
            raise ValueError(f"packed_weight shape {tuple(packed_weight.shape)} != ({out_features}, {in_features // 4})")
        return ops.bitlinear(x.to(self.compute_dtype), packed_weight, scale, bias=bias, layout=self.layout,
                             out_dtype=self.compute_dtype)

    def clear_cache(self):  # the reference caches dequantized weights; nothing is cached here
        pass


class BitNetLinearNative(nn.Module):
    """Linear layer on packed 2-bit weights (I2_S layout by default)."""

    def __init__(self, in_features: int, out_features: int, packed_weight: torch.Tensor, weight_scale: torch.Tensor,
                 bias: Optional[torch.Tensor] = None, layout: int = L.LAYOUT_I2S):
        super().__init__()
        self.in_features, self.out_features, self.layout = in_features, out_features, layout
        self.register_buffer("packed_weight", packed_weight)
        self.register_buffer("weight_scale", weight_scale.reshape(-1).to(torch.float32))
        if bias is not None:
            self.register_buffer("bias", bias)
        else:
            self.bias = None

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return ops.bitlinear(x, self.packed_weight, self.weight_scale, bias=self.bias, layout=self.layout,
                             out_dtype=torch.float32 if x.dtype == torch.float32 else x.dtype)
