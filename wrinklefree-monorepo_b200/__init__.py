"""wf_b200: B200-native (sm_100a) ternary BitLinear — packed 2-bit absmean weights,
per-token int8 activations, int32 accumulation, fp32 rescale — behind the
reference's module and operator interfaces.  CUDA only; no CPU fallback."""
from . import _lib  # noqa: F401
from .bitlinear import BitLinear, BitLinearNoActivationQuant, convert_linear_to_bitlinear  # noqa: F401
from .lambda_warmup import (  # noqa: F401
    LambdaWarmup,
    get_current_lambda,
    get_global_lambda_warmup,
    set_global_lambda_warmup,
)
from .convert import (  # noqa: F401
    RMSNorm,
    SubLN,
    convert_attention_layer,
    convert_mlp_layer,
    convert_model_to_bitnet,
)
from .linear_method import (  # noqa: F401
    BitNetConfig,
    BitNetLinearMethod,
    BitNetLinearNative,
    PackedBitNetLinearMethod,
    create_bitnet_config,
    dequantize_bitnet,
    pack_ternary_weights,
    patch_model_with_native_kernels,
    quantize_to_bitnet,
)
from .ops import (  # noqa: F401
    QK_I2_S,
    DecodeGroup,
    device_status,
    act_quant_i8,
    bitlinear,
    bitlinear_batched,
    bitnet_gemm,
    bitnet_gemv,
    check_kernel_available,
    linear_bf16,
    pack_codes,
    pack_ternary,
    prefill_quantize,
    prefill_workspace,
    quantize_activations_i8,
    quantize_maxabs,
    repack,
    stack_uses_contraction,
    unpack_codes,
)
from . import torch_ops  # noqa: F401,E402  (registers torch.ops.wf_b200.*)
