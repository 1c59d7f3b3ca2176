"""The inference side's "ternary linear method", with the reference's signatures.

* ``BitNetConfig`` / ``BitNetLinearMethod``: the SGLang quantization plug-in
  (sglang/srt/layers/quantization/bitnet.py:45-255): ``create_weights``,
  ``process_weights_after_loading``, ``apply(layer, x, bias)``.  SGLang itself is
  not needed to import this module; when it is installed the classes can be
  registered under the name "bitnet" unchanged.
* ``PackedBitNetLinearMethod``: the first-party twin whose ``apply`` takes the
  packed weight explicitly (wrinklefree_inference/sglang_backend/bitnet_quantization.py:366-409).
* ``BitNetLinearNative``: the patched module (wrinklefree_inference/kernels/bitnet_patch.py:28-78).

The SGLang plug-in's weights arrive in the I2_S block layout, as checkpoints of
the reference store them; the kernels consume that layout directly.  The two
first-party classes take the byte orders of their own packers (sequential,
MSB-first and LSB-first) and convert once.  No host synchronisation happens in
``apply`` (the reference calls ``scale.item()`` per call).
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


def _kernel_copy(packed: torch.Tensor, layout: int, n: int, k: int) -> torch.Tensor:
    """Packed weights in a layout the kernels consume: WF16 / I2S as they are, the sequential and HF
    layouts converted once on the GPU."""
    if layout in (L.LAYOUT_WF16, L.LAYOUT_I2S):
        return packed if packed.is_contiguous() else packed.contiguous()
    return ops.repack(packed, layout, n, k, L.LAYOUT_WF16)


class PackedBitNetLinearMethod:
    """First-party signature: apply(packed_weight, scale, x, out_features, in_features, bias)
    (wrinklefree_inference/sglang_backend/bitnet_quantization.py:366-409).

    `packed_weight` holds the bytes that interface's own packer emits: `quantize_to_bitnet` writes four consecutive
    weights per byte, first weight in the top bit pair (L.LAYOUT_SEQ_MSB), which is the default here.  The bytes are
    converted to the kernels' layout once per tensor and the copy is cached (keyed like the reference's cache of
    dequantized weights, by tensor identity; `clear_cache` drops it).  Activations are quantized to int8 per token
    (W2A8), where the reference multiplies dequantized weights in bf16."""

    def __init__(self, compute_dtype: torch.dtype = torch.bfloat16, layout: int = L.LAYOUT_SEQ_MSB):
        self.compute_dtype = compute_dtype
        self.layout = layout
        self._cache: Dict[tuple, torch.Tensor] = {}

    def _kernel_weight(self, packed: torch.Tensor, n: int, k: int) -> torch.Tensor:
        key = (packed.data_ptr(), packed._version, n, k, packed.device)
        hit = self._cache.get(key)
        if hit is None:
            hit = _kernel_copy(packed, self.layout, n, k)
            self._cache[key] = hit
        return hit

    def apply(self, packed_weight: torch.Tensor, scale, x: torch.Tensor, out_features: int, in_features: int,
              bias: Optional[torch.Tensor] = None, sparsity_config=None) -> torch.Tensor:
        if sparsity_config is not None and getattr(sparsity_config, "enabled", False):
            raise NotImplementedError("activation sparsity is not part of the CUDA path")
        if packed_weight.shape != (out_features, in_features // 4):
            raise ValueError(f"packed_weight shape {tuple(packed_weight.shape)} != ({out_features}, {in_features // 4})")
        codes = self._kernel_weight(packed_weight, out_features, in_features)
        lay = self.layout if self.layout in (L.LAYOUT_WF16, L.LAYOUT_I2S) else L.LAYOUT_WF16
        return ops.bitlinear(x.to(self.compute_dtype), codes, scale, bias=bias, layout=lay, out_dtype=self.compute_dtype)

    def clear_cache(self):
        self._cache.clear()


def quantize_to_bitnet(weights: torch.Tensor, block_size: int = BITNET_BLOCK_SIZE):
    """GPU twin of quantize_to_bitnet (sglang_backend/bitnet_quantization.py:69-109): (packed uint8 [N, K/4] in the
    SEQ_MSB byte order, scale = max|w| as a float32 tensor [1] on the device - no host synchronisation)."""
    if weights.shape[1] % block_size != 0:
        raise ValueError(f"in_features must be divisible by {block_size}")
    return ops.quantize_maxabs(weights, "half", L.LAYOUT_SEQ_MSB)


def dequantize_bitnet(packed: torch.Tensor, scale, out_features: int, in_features: int,
                      layout: int = L.LAYOUT_SEQ_MSB) -> torch.Tensor:
    """float32 [N, K] = ternary * scale (sglang_backend/bitnet_quantization.py:211-252), unpacked on the GPU."""
    t = ops.unpack_codes(packed, out_features, in_features, layout).to(torch.float32)
    return t * (scale if isinstance(scale, torch.Tensor) else float(scale))


def pack_ternary_weights(weight: torch.Tensor):
    """GPU twin of pack_ternary_weights (wrinklefree_inference/kernels/bitnet_patch.py:81-112): rounds to
    {-1, 0, 1}, packs four consecutive weights per byte, first weight in the low bit pair (L.LAYOUT_SEQ_LSB);
    scale = max|w| (below 1e-6: 1) as a float32 device tensor."""
    if weight.shape[1] % 4 != 0:
        raise ValueError(f"in_features ({weight.shape[1]}) must be divisible by 4")
    t = torch.round(weight.float()).clamp_(-1, 1).to(torch.int8)
    mx = weight.abs().max().float()
    return ops.pack_codes(t, L.LAYOUT_SEQ_LSB), torch.where(mx < 1e-6, torch.ones_like(mx), mx)


class BitNetLinearNative(nn.Module):
    """Linear layer on packed 2-bit weights (wrinklefree_inference/kernels/bitnet_patch.py:28-78).  `packed_weight`
    arrives in the byte order of the packer that sits next to that class, `pack_ternary_weights` (L.LAYOUT_SEQ_LSB);
    pass layout=L.LAYOUT_I2S for checkpoints in the block layout.  A kernel-layout copy is made once at construction;
    the original bytes stay in the `packed_weight` buffer (state_dict compatible)."""

    def __init__(self, in_features: int, out_features: int, packed_weight: torch.Tensor, weight_scale: torch.Tensor,
                 bias: Optional[torch.Tensor] = None, layout: int = L.LAYOUT_SEQ_LSB, act_quant: str = "per_token"):
        super().__init__()
        self.in_features, self.out_features, self.layout, self.act_quant = in_features, out_features, layout, act_quant
        self.register_buffer("packed_weight", packed_weight)
        self.register_buffer("weight_scale", weight_scale.reshape(-1).to(torch.float32))
        if bias is not None:
            self.register_buffer("bias", bias)
        else:
            self.bias = None
        self._kernel = None  # (key, codes in a kernel layout)

    def _codes(self) -> torch.Tensor:
        pw = self.packed_weight
        key = (pw.data_ptr(), pw._version, pw.device)
        if self._kernel is None or self._kernel[0] != key:
            self._kernel = (key, _kernel_copy(pw, self.layout, self.out_features, self.in_features))
        return self._kernel[1]

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        lay = self.layout if self.layout in (L.LAYOUT_WF16, L.LAYOUT_I2S) else L.LAYOUT_WF16
        out_dtype = torch.float32 if x.dtype == torch.float32 else x.dtype
        if self.act_quant == "per_tensor":  # the arithmetic of the class this mirrors: one scale for the whole batch
            q, s = ops.quantize_activations_i8(x.reshape(-1, self.in_features))
            out = ops.bitlinear(q, self._codes(), self.weight_scale, layout=lay, out_dtype=torch.float32) * s
            out = out + self.bias if self.bias is not None else out
            return out.to(out_dtype).reshape(*x.shape[:-1], self.out_features)
        return ops.bitlinear(x, self._codes(), self.weight_scale, bias=self.bias, layout=lay, out_dtype=out_dtype)


def patch_model_with_native_kernels(model: nn.Module) -> int:
    """Replaces every linear-like module that carries packed uint8 weights (attribute `weight` of dtype uint8 with a
    `weight_scale` or `scale`) or float weights that are already ternary by a BitNetLinearNative
    (wrinklefree_inference/kernels/bitnet_patch.py:165-210).  Returns the number of modules replaced."""
    if not ops.check_kernel_available():
        return 0
    patched = 0
    for name, module in list(model.named_modules()):
        if not (isinstance(module, nn.Linear) or "Linear" in type(module).__name__) or isinstance(module, BitNetLinearNative):
            continue
        w = getattr(module, "weight", None)
        if w is None or w.numel() == 0:
            continue
        w = w.data
        if w.dtype == torch.uint8:
            packed = w
            sc = getattr(module, "weight_scale", None)
            sc = sc if sc is not None else getattr(module, "scale", None)
            scale = sc.data if sc is not None else torch.ones(1, device=w.device)
        else:
            r = torch.round(w.float())
            if not bool(((r.abs() <= 1) & ((w.float() - r).abs() < 1e-6)).all()):
                continue  # not ternary: left alone, as the reference does
            packed, scale = pack_ternary_weights(w)  # max|w| of ternary values is 1 (all-zero: 1 as well)
            scale = scale.reshape(1)
        n, k = packed.shape[0], packed.shape[1] * 4
        if k % BITNET_BLOCK_SIZE != 0:
            continue
        bias = module.bias.data if getattr(module, "bias", None) is not None else None
        native = BitNetLinearNative(k, n, packed, scale.to(w.device), bias)
        parent = model.get_submodule(".".join(name.split(".")[:-1])) if "." in name else model
        setattr(parent, name.split(".")[-1], native)
        patched += 1
    return patched


def create_bitnet_config(**kwargs) -> BitNetConfig:
    """Factory kept from sglang/srt/layers/quantization/bitnet.py:259-261."""
    return BitNetConfig(**kwargs)
