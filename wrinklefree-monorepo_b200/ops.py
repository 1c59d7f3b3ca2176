"""Tensor-level wrappers over the C ABI, plus the operator API of the reference's
sgl_kernel.quantization.bitnet module under the same names.

All tensors must live on a CUDA device of compute capability 10.x; the current
torch stream is used.  Nothing here computes on the CPU.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch

from . import _lib as L

QK_I2_S = 128  # block size of the I2_S layout (sgl_kernel/quantization/bitnet.py:14)

_DT = {torch.float32: L.WF_F32, torch.float16: L.WF_F16, torch.bfloat16: L.WF_BF16, torch.int8: L.WF_I8}
_PACK_MODE = {torch.float32: L.PACK_FP32, torch.bfloat16: L.PACK_CAST_BF16, torch.float16: L.PACK_CAST_F16}
DECODE_MAX_TOKENS = 64  # token counts above this go to the prefill entry point


def stack_uses_contraction(m: int, k: int) -> bool:
    """Which kernel a STACK of independent same-shape layers with `m` tokens each should run on: the batched tensor-core
    contraction (`bitlinear_batched`) or the grouped streaming launch (`DecodeGroup`).  Measured on B200 on stacks of
    16 to 120 layers (2560x2560, 6912x2560, 2560x6912, 4096x4096, 4096x14336; the contraction timed with its
    quantization kernel): the contraction's time does not depend on m up to 16 tokens, the streaming kernel's grows
    with m (its legacy MMA covers 8 tokens per instruction, and activations of long rows crowd its stages out of
    shared memory); they cross at 2 to 4 tokens for K >= 4096 and between 4 and 8 tokens for K = 2560."""
    return m >= 8 or (m >= 4 and k >= 4096)


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _need_cuda(*ts):
    for t in ts:
        if t is not None and not t.is_cuda:
            raise RuntimeError("wf_b200 operators need CUDA tensors (there is no CPU path)")


def _ptr(t: Optional[torch.Tensor]):
    return None if t is None else t.data_ptr()


def check_kernel_available() -> bool:
    """True when the compiled library is loadable and the current device is sm_100
    (name kept from sgl_kernel/quantization/bitnet.py:39-45)."""
    try:
        return torch.cuda.is_available() and L.lib().wf_device_check() == 0
    except (RuntimeError, OSError):
        return False


# --------------------------------------------------------------------------
# weights
# --------------------------------------------------------------------------


def pack_ternary(weight: torch.Tensor, mode: torch.dtype = torch.float32, eps: float = 1e-5
                 ) -> Tuple[torch.Tensor, torch.Tensor]:
    """Absmean-ternarize `weight` [N, K] and pack it 2 bits per weight (WF16 layout).

    mode torch.float32: scale = mean|w| in fp32, codes = clamp(round(w / scale)) as
    ternary_weight_quantization_no_scale (wrinklefree/quantization/weight_quant.py:35-56).
    mode torch.bfloat16 / torch.float16: the cast-first arithmetic that BitLinear.forward
    applies when its input has that dtype (wrinklefree/models/bitlinear.py:103-107).
    Returns (codes uint8 [N, K/4], scale float32 [2]): scale[0] is the dequantization
    multiplier, scale[1] the quantization multiplier.
    """
    _need_cuda(weight)
    if weight.dim() != 2:
        raise ValueError("pack_ternary expects a 2-D weight")
    if weight.stride(1) != 1:
        weight = weight.contiguous()
    n, k = weight.shape
    lib = L.lib()
    codes = torch.empty((n, k // 4), dtype=torch.uint8, device=weight.device)
    scale = torch.empty(2, dtype=torch.float32, device=weight.device)
    nbytes = lib.wf_pack_scratch_bytes(n, k)
    scratch = torch.empty(max(nbytes, 8), dtype=torch.uint8, device=weight.device)
    with torch.cuda.device(weight.device):
        L.check(lib.wf_pack_ternary(weight.data_ptr(), _DT[weight.dtype], n, k, weight.stride(0), _PACK_MODE[mode], eps,
                                    codes.data_ptr(), scale.data_ptr(), scratch.data_ptr(), scratch.numel(), _stream()),
                "wf_pack_ternary")
    return codes, scale


def repack(src: torch.Tensor, src_layout: int, n: int, k: int, dst_layout: int = L.LAYOUT_WF16) -> torch.Tensor:
    """Convert packed ternary weights between layouts on the GPU (constants L.LAYOUT_*)."""
    _need_cuda(src)
    src = src.contiguous()
    if src.numel() != n * k // 4:
        raise ValueError(f"packed tensor has {src.numel()} bytes, expected {n * k // 4}")
    dst = torch.empty((n, k // 4), dtype=torch.uint8, device=src.device)
    with torch.cuda.device(src.device):
        L.check(L.lib().wf_repack(src.data_ptr(), src_layout, dst.data_ptr(), dst_layout, n, k, _stream()), "wf_repack")
    return dst


def quantize_maxabs(weight: torch.Tensor, rule: str = "half", layout: int = L.LAYOUT_SEQ_MSB) -> Tuple[torch.Tensor, torch.Tensor]:
    """The max-abs quantizers of the inference side on the GPU: returns (packed uint8 [N, K/4] in `layout`,
    scale float32 [1] = max|w|).  rule "half": codes by thresholds at +-0.5 of w / max (quantize_to_bitnet,
    sglang_backend/bitnet_quantization.py:69-109, whose bytes are SEQ_MSB); rule "sign": codes by sign with a
    1e-6 dead zone (quantize_i2_s, BitNet/src/ggml-bitnet-mad.cpp:46-92, whose bytes are I2S)."""
    _need_cuda(weight)
    if weight.dim() != 2:
        raise ValueError("quantize_maxabs expects a 2-D weight")
    if weight.stride(1) != 1:
        weight = weight.contiguous()
    n, k = weight.shape
    codes = torch.empty((n, k // 4), dtype=torch.uint8, device=weight.device)
    scale = torch.empty(2, dtype=torch.float32, device=weight.device)
    with torch.cuda.device(weight.device):
        L.check(L.lib().wf_quantize_maxabs(weight.data_ptr(), _DT[weight.dtype], n, k, weight.stride(0),
                                           L.MAXABS_HALF if rule == "half" else L.MAXABS_SIGN, layout, codes.data_ptr(),
                                           scale.data_ptr(), _stream()), "wf_quantize_maxabs")
    return codes, scale[:1]


def pack_codes(ternary: torch.Tensor, layout: int = L.LAYOUT_WF16) -> torch.Tensor:
    """Pack int8 values in {-1, 0, 1} [N, K] into a kernel layout."""
    _need_cuda(ternary)
    t = ternary.to(torch.int8).contiguous()
    n, k = t.shape
    dst = torch.empty((n, k // 4), dtype=torch.uint8, device=t.device)
    with torch.cuda.device(t.device):
        L.check(L.lib().wf_pack_codes(t.data_ptr(), dst.data_ptr(), layout, n, k, _stream()), "wf_pack_codes")
    return dst


def unpack_codes(packed: torch.Tensor, n: int, k: int, layout: int = L.LAYOUT_WF16) -> torch.Tensor:
    _need_cuda(packed)
    packed = packed.contiguous()
    out = torch.empty((n, k), dtype=torch.int8, device=packed.device)
    with torch.cuda.device(packed.device):
        L.check(L.lib().wf_unpack_codes(packed.data_ptr(), layout, out.data_ptr(), n, k, _stream()), "wf_unpack_codes")
    return out


# --------------------------------------------------------------------------
# activations
# --------------------------------------------------------------------------


def act_quant_i8(x: torch.Tensor, per_tensor: bool = False, eps: float = 1e-5, want_rowsum: bool = False):
    """int8 activation quantization.  Per token (default) follows BitLinear.activation_quant
    in the arithmetic of x.dtype; per_tensor follows bitnet_quantize_activations_cpu (fp32).
    Returns (q int8 same shape, scale fp32 [M] or [1][, rowsum int32 [M]])."""
    _need_cuda(x)
    k = x.shape[-1]
    x2 = x.reshape(-1, k)
    if x2.stride(1) != 1:
        x2 = x2.contiguous()
    m = x2.shape[0]
    q = torch.empty((m, k), dtype=torch.int8, device=x.device)
    scale = torch.empty(1 if per_tensor else m, dtype=torch.float32, device=x.device)
    rowsum = torch.empty(m, dtype=torch.int32, device=x.device) if want_rowsum else None
    with torch.cuda.device(x.device):
        L.check(L.lib().wf_act_quant_i8(x2.data_ptr(), _DT[x2.dtype], m, k, x2.stride(0),
                                        L.ACT_PER_TENSOR if per_tensor else L.ACT_PER_TOKEN, eps, q.data_ptr(),
                                        scale.data_ptr(), _ptr(rowsum), _stream()), "wf_act_quant_i8")
    q = q.reshape(x.shape)
    return (q, scale, rowsum) if want_rowsum else (q, scale)


# --------------------------------------------------------------------------
# the contraction
# --------------------------------------------------------------------------

_workspaces = {}
# Decode path: every CTA of the decode kernel quantizes the tokens of its problem itself.  That is the right trade for a
# stack of many small problems (a CTA meets one or two of them), not for one projection that all CTAs share: there a
# quantization kernel in front (same arithmetic, same bits) takes the absmax reduction and its barriers off the critical
# path of every CTA.  Measured on the 8B shape: 63.6 -> 61.0 us per layer at one sequence, 87.7 -> 68.6 at four,
# 118.5 -> 86.6 at eight.
PREQUANT_MIN_TOKENS = 16    # any launch: tokens per problem from which x is quantized once by a kernel of its own
PREQUANT_MIN_ELEMS = 4096   # launches of at most PREQUANT_MAX_PROBLEMS problems: tokens x K from which it is
PREQUANT_MAX_PROBLEMS = 4


def _prequant(m: int, k: int, problems: int = 1) -> bool:
    return m >= PREQUANT_MIN_TOKENS or (problems <= PREQUANT_MAX_PROBLEMS and m * k >= PREQUANT_MIN_ELEMS)


def _workspace(device, nbytes: int) -> torch.Tensor:
    ws = _workspaces.get(device)
    if ws is None or ws.numel() < nbytes:
        ws = torch.empty(max(nbytes, 1 << 20), dtype=torch.uint8, device=device)
        _workspaces[device] = ws
    return ws


def bitlinear(x: torch.Tensor, codes: torch.Tensor, w_scale, bias: Optional[torch.Tensor] = None,
              out_dtype: Optional[torch.dtype] = None, layout: int = L.LAYOUT_WF16, x_scale: Optional[torch.Tensor] = None,
              eps: float = 1e-5, want_acc: bool = False, pdl: bool = False, path: str = "auto",
              out: Optional[torch.Tensor] = None, prefill_form: str = "auto"):
    """y = BitLinear(x) on packed weights: per-token int8 quantization of x (fused for small
    token counts), exact int32 contraction with the ternary codes, fp32 rescale
    ``(float(acc) * (1/s_x[m])) * s_w`` and optional bias.

    x: [..., K] float32/float16/bfloat16, or int8 (already quantized; x_scale [M] optional).
    codes: uint8 [N, K/4] in `layout`.  w_scale: device tensor (first element used) or float.
    path: "auto" (decode kernel for few tokens, the tensor-core contraction otherwise), "decode" or "prefill".
    prefill_form: "auto", or "pair" / "single" to force the two-SM or the one-SM tile form of the contraction.
    Returns y [..., N] (and the int32 accumulators [M, N] when want_acc).
    """
    _need_cuda(x, codes, bias, x_scale)
    k = x.shape[-1]
    n = codes.shape[0]
    if codes.dtype != torch.uint8 or codes.dim() != 2 or codes.shape[1] * 4 != k:
        raise ValueError(f"codes must be uint8 [N, K/4] with K={k}, got {tuple(codes.shape)} {codes.dtype}")
    x2 = x.reshape(-1, k)
    if x2.stride(1) != 1:
        x2 = x2.contiguous()
    m = x2.shape[0]
    if out_dtype is None:
        out_dtype = torch.float32 if x.dtype == torch.int8 else x.dtype
    y = out if out is not None else torch.empty((m, n), dtype=out_dtype, device=x.device)
    acc = torch.empty((m, n), dtype=torch.int32, device=x.device) if want_acc else None
    if isinstance(w_scale, torch.Tensor):
        ws_ptr, ws_host = w_scale.data_ptr(), 0.0
        if w_scale.dtype != torch.float32 or not w_scale.is_cuda:
            raise ValueError("w_scale tensor must be float32 on the GPU")
    else:
        ws_ptr, ws_host = None, float(w_scale)
    if not codes.is_contiguous():
        codes = codes.contiguous()
    lib = L.lib()
    flags = L.FLAG_PDL if pdl else 0
    flags |= {"auto": 0, "pair": L.FLAG_PREFILL_PAIR, "single": L.FLAG_PREFILL_SINGLE}[prefill_form]
    # auto: the tensor-core contraction above DECODE_MAX_TOKENS tokens, and from 16 tokens on for matrices of at least
    # 4 Mi weights (measured: 4096 x 4096 at 32 tokens 14 us against 20 us on the decode kernel; small layers the reverse)
    use_prefill = path == "prefill" or (path == "auto" and (m > DECODE_MAX_TOKENS or (m >= 16 and n * k >= (1 << 22))))
    with torch.cuda.device(x.device):
        if m == 0:
            pass
        elif use_prefill:
            nbytes = lib.wf_prefill_workspace_bytes(m, k)
            ws = _workspace(x.device, nbytes)
            L.check(lib.wf_bitlinear_prefill(x2.data_ptr(), _DT[x2.dtype], x2.stride(0), _ptr(x_scale), codes.data_ptr(),
                                             layout, ws_ptr, ws_host, _ptr(bias), _DT[bias.dtype] if bias is not None else 0,
                                             y.data_ptr(), _DT[y.dtype], y.stride(0), _ptr(acc), m, n, k, eps,
                                             _ptr(ws), ws.numel() if ws is not None else 0, flags, _stream()),
                    "wf_bitlinear_prefill")
        else:
            if x2.dtype != torch.int8 and _prequant(m, k):
                # every CTA of the decode kernel quantizes the tokens of its problem: from this many tokens on one
                # quantization kernel in front of it is cheaper (same arithmetic, same bits)
                x2, x_scale = act_quant_i8(x2, eps=eps)
            L.check(lib.wf_bitlinear_decode(x2.data_ptr(), _DT[x2.dtype], x2.stride(0), _ptr(x_scale), codes.data_ptr(),
                                            layout, ws_ptr, ws_host, _ptr(bias), _DT[bias.dtype] if bias is not None else 0,
                                            y.data_ptr(), _DT[y.dtype], y.stride(0), _ptr(acc), m, n, k, eps, flags,
                                            _stream()), "wf_bitlinear_decode")
    y = y.reshape(*x.shape[:-1], n)
    return (y, acc) if want_acc else y


def prefill_workspace(m_rows: int, k: int, device) -> torch.Tensor:
    """A workspace of its own for `m_rows` tokens of width `k` (see `prefill_quantize`)."""
    return torch.empty(L.lib().wf_prefill_workspace_bytes(m_rows, k), dtype=torch.uint8, device=device)


def prefill_quantize(x: torch.Tensor, workspace: torch.Tensor, eps: float = 1e-5, independent: bool = False) -> None:
    """Quantizes the tokens x [..., K] (per-token absmax int8, scales, row sums) into `workspace`
    (`prefill_workspace(tokens, K, device)`): the first half of `bitlinear_batched`, for calls with `workspace=` and
    `quantized=True`.  One quantization serves every projection of the same tokens.  `independent=True`: no kernel that
    may still be running writes x or uses the workspace, so the launch need not wait for its predecessor."""
    _need_cuda(x, workspace)
    k = x.shape[-1]
    x2 = x.reshape(-1, k)
    if x2.stride(1) != 1:
        raise ValueError("prefill_quantize needs x with unit inner stride")
    with torch.cuda.device(x.device):
        L.check(L.lib().wf_prefill_quantize(x2.data_ptr(), _DT[x.dtype], x2.stride(0), x2.shape[0], k, eps, workspace.data_ptr(),
                                            workspace.numel(), L.FLAG_X_READY if independent else 0, _stream()),
                "wf_prefill_quantize")


def bitlinear_batched(x: torch.Tensor, codes: torch.Tensor, w_scales: torch.Tensor, out: Optional[torch.Tensor] = None,
                      out_dtype: Optional[torch.dtype] = None, layout: int = L.LAYOUT_WF16, eps: float = 1e-5,
                      want_acc: bool = False, workspace: Optional[torch.Tensor] = None, quantized: bool = False,
                      independent: bool = False):
    """A stack of `B` independent BitLinear layers of one shape in one tensor-core launch.

    x [B, M, K] (contiguous), codes uint8 [B, N, K/4] (contiguous), w_scales float32 [B] or [B, 2] (first column used).
    Returns y [B, M, N] (and the int32 accumulators when want_acc).

    `workspace` (default: one shared per device) with `quantized=True`: `prefill_quantize(x, workspace)` ran earlier in
    the stream and x is not read again.  `independent=True` in addition: the workspace and the output have nothing to do
    with the launches since the last contraction that was not marked so (the quantizations went first, then one
    unmarked contraction): the launch does not wait for its predecessor and fills the SMs its tail leaves idle.
    """
    _need_cuda(x, codes, w_scales)
    b, m, k = x.shape
    n = codes.shape[1]
    if codes.shape != (b, n, k // 4) or not codes.is_contiguous() or not x.is_contiguous():
        raise ValueError("bitlinear_batched needs contiguous x [B, M, K] and codes [B, N, K/4]")
    if w_scales.dtype != torch.float32 or w_scales.shape[0] != b:
        raise ValueError("w_scales must be float32 with one row per layer")
    if (quantized or independent) and workspace is None:
        raise ValueError("quantized / independent need the workspace that prefill_quantize filled")
    if independent and not quantized:
        raise ValueError("independent=True needs quantized=True")
    y = out if out is not None else torch.empty((b, m, n), dtype=out_dtype or x.dtype, device=x.device)
    if not y.is_contiguous():
        raise ValueError("out must be contiguous")
    acc = torch.empty((b * m, n), dtype=torch.int32, device=x.device) if want_acc else None
    lib = L.lib()
    nbytes = lib.wf_prefill_workspace_bytes(b * m, k)
    ws = workspace if workspace is not None else _workspace(x.device, nbytes)
    flags = (L.FLAG_WS_READY if quantized else 0) | (L.FLAG_X_READY if independent else 0)
    with torch.cuda.device(x.device):
        L.check(lib.wf_bitlinear_prefill_batched(x.data_ptr(), _DT[x.dtype], k, codes.data_ptr(), layout, w_scales.data_ptr(),
                                                 w_scales.stride(0), y.data_ptr(), _DT[y.dtype], n, _ptr(acc), b, m, n, k, eps,
                                                 ws.data_ptr(), ws.numel(), flags, _stream()), "wf_bitlinear_prefill_batched")
    return (y, acc.view(b, m, n)) if want_acc else y


class DecodeGroup:
    """Several independent BitLinear problems run as one persistent kernel (q/k/v, gate/up, or a
    stack of layers).  Build once, `run()` any number of times; the tensors given at construction
    are read / written in place on every run.

    problems: iterable of dicts with keys x, codes, w_scale and optionally bias, out, out_dtype,
    layout, x_scale, eps, want_acc.  All x must share a dtype.

    `prefetch`: a tensor whose bytes the launch asks L2 to fetch while it runs (the next launch's packed weights).

    `xchg`: the device pointer of an exchange (`tp.OneShotAllReduce.xchg_ptr()`): a row-parallel projection pushes its
    partial output to every rank inside the launch; `OneShotAllReduce.reduce_add_rmsnorm_` consumes it.

    Fused inputs (bf16): `x_mode` "silu" / "relu2" with `x2`: the projection quantizes act(x) * x2 (x = gate,
    x2 = up: the activation in front of a down projection); `x_mode` "norm" with `norm_w`, optional `x2`, `h_out`,
    `norm_eps`: it quantizes rmsnorm(x + x2) * norm_w and writes x + x2 to h_out (residual add + RMSNorm in front
    of q/k/v or gate/up).  The arithmetic is that of `act_mul` / `add_rmsnorm_`, so a fused launch replaces the
    separate kernel.
    """

    _XMODE = {None: L.X_PLAIN, "plain": L.X_PLAIN, "silu": L.X_SILU, "relu2": L.X_RELU2, "norm": L.X_NORM}

    def __init__(self, problems):
        import ctypes as C

        problems = list(problems)
        if not problems:
            raise ValueError("empty group")
        self._keep = []
        self.outputs, self.accs = [], []
        self.x_ptr = None  # address of the first pushing problem's input (a caller may have to copy into it)
        arr, self._raw = L.aligned_problem_array(len(problems))
        dev = problems[0]["x"].device
        # With many tokens per problem x is quantized once per distinct input by a kernel of its own in run(), and
        # the problems read the int8 copy (otherwise every CTA quantizes the tokens of its problem again).
        prequant = all(pr["x"].dtype != torch.int8 and _prequant(pr["x"].reshape(-1, pr["x"].shape[-1]).shape[0], pr["x"].shape[-1], len(problems))
                       and not pr.get("x_mode") for pr in problems)
        self._quant = {}  # data_ptr of x -> (x2, q, scale, eps)
        for i, pr in enumerate(problems):
            x, codes, w_scale = pr["x"], pr["codes"], pr["w_scale"]
            bias, x_scale = pr.get("bias"), pr.get("x_scale")
            _need_cuda(x, codes, bias, x_scale)
            k = x.shape[-1]
            x2 = x.reshape(-1, k)
            if x2.stride(1) != 1 or not codes.is_contiguous():
                raise ValueError("DecodeGroup needs x with unit inner stride and contiguous codes")
            m, n = x2.shape[0], codes.shape[0]
            out_dtype = pr.get("out_dtype") or (torch.float32 if x.dtype == torch.int8 else x.dtype)
            if prequant:
                key = (x2.data_ptr(), x2.stride(0), m, k, pr.get("eps", 1e-5))
                if key not in self._quant:
                    self._quant[key] = (x2, torch.empty((m, k), dtype=torch.int8, device=dev),
                                        torch.empty(m, dtype=torch.float32, device=dev), pr.get("eps", 1e-5))
                _, x2, x_scale, _ = self._quant[key]
            y = pr.get("out")
            if y is None:
                y = torch.empty((m, n), dtype=out_dtype, device=dev)
            acc = torch.empty((m, n), dtype=torch.int32, device=dev) if pr.get("want_acc") else None
            q = arr[i]
            q.x, q.x_scale, q.codes = x2.data_ptr(), _ptr(x_scale), codes.data_ptr()
            if isinstance(w_scale, torch.Tensor):
                q.w_scale, q.w_scale_host = w_scale.data_ptr(), 0.0
            else:
                q.w_scale, q.w_scale_host = None, float(w_scale)
            q.bias, q.y, q.acc_out = _ptr(bias), y.data_ptr(), _ptr(acc)
            q.ldx, q.ldy, q.M, q.N, q.K = x2.stride(0), y.stride(0), m, n, k
            q.x_dtype, q.y_dtype = _DT[x2.dtype], _DT[y.dtype]
            q.bias_dtype = _DT[bias.dtype] if bias is not None else 0
            q.layout, q.eps = pr.get("layout", L.LAYOUT_WF16), pr.get("eps", 1e-5)
            mode = self._XMODE[pr.get("x_mode")]
            if mode != L.X_PLAIN:
                second, norm_w, h_out = pr.get("x2"), pr.get("norm_w"), pr.get("h_out")
                _need_cuda(second, norm_w, h_out)
                for t_ in (second, h_out):
                    if t_ is not None and (t_.dtype != x.dtype or t_.reshape(-1, k).stride(0) != x2.stride(0)):
                        raise ValueError("x2 / h_out must have the dtype and row stride of x")
                q.x_mode, q.norm_eps = mode, pr.get("norm_eps", 1e-6)
                q.x2, q.norm_w, q.h_out = _ptr(second), _ptr(norm_w), _ptr(h_out)
                self._keep += [second, norm_w, h_out]
            if pr.get("xchg"):  # device pointer of an exchange (tp.OneShotAllReduce.xchg_ptr()): the launch pushes this output
                q.xchg = int(pr["xchg"])
                if self.x_ptr is None:
                    self.x_ptr = x.reshape(-1, k).data_ptr()  # the caller's tensor, also when an int8 copy is what the kernel reads
            pf = pr.get("prefetch")  # a tensor (typically the next launch's packed weights) to pull into L2 meanwhile
            if pf is not None:
                _need_cuda(pf)
                q.prefetch, q.prefetch_bytes = pf.data_ptr(), pf.numel() * pf.element_size() // 16 * 16
                self._keep.append(pf)
            self._keep += [x2, codes, w_scale, bias, x_scale, y, acc]
            self.outputs.append(y.reshape(*x.shape[:-1], n))
            self.accs.append(acc)
        self.device = dev
        self._host = arr
        with torch.cuda.device(dev):
            L.check(L.lib().wf_bitlinear_decode_plan(C.addressof(arr), len(problems)), "wf_bitlinear_decode_plan")
        raw = bytes(arr)
        self._dev = torch.frombuffer(bytearray(raw), dtype=torch.uint8).to(dev)
        self.count = len(problems)

    def run(self, pdl: bool = False, x_ready: bool = False):
        """Launches the group.  `x_ready` (with `pdl`): the inputs were not written by the previous kernel of the
        stream, so the kernel reads them without waiting for it (independent layers, experts, replicas)."""
        import ctypes as C

        flags = (L.FLAG_PDL if pdl else 0) | (L.FLAG_X_READY if (pdl and x_ready and not self._quant) else 0)
        with torch.cuda.device(self.device):
            for (xs, q, scale, eps) in self._quant.values():
                L.check(L.lib().wf_act_quant_i8(xs.data_ptr(), _DT[xs.dtype], xs.shape[0], xs.shape[1], xs.stride(0),
                                                L.ACT_PER_TOKEN, eps, q.data_ptr(), scale.data_ptr(), None, _stream()),
                        "wf_act_quant_i8")
            L.check(L.lib().wf_bitlinear_decode_grouped(self._dev.data_ptr(), C.addressof(self._host), self.count,
                                                        flags, _stream()), "wf_bitlinear_decode_grouped")
        return self.outputs


def add_rmsnorm_(h: torch.Tensor, delta: Optional[torch.Tensor], weight: torch.Tensor, out: torch.Tensor, eps: float,
                 pdl: bool = False):
    """h += delta (if given), out = rmsnorm(h) * weight; bf16, contiguous [M, K].  `pdl`: chain the launch to its
    neighbours in the stream with a programmatic dependency (same meaning for the other kernels of this group)."""
    _need_cuda(h, delta, weight, out)
    m, k = h.shape
    with torch.cuda.device(h.device):
        L.check(L.lib().wf_add_rmsnorm_bf16(h.data_ptr(), _ptr(delta), weight.data_ptr(), out.data_ptr(), m, k, eps,
                                            L.FLAG_PDL if pdl else 0, _stream()), "wf_add_rmsnorm_bf16")
    return out


def rope_kv_(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, pos: torch.Tensor,
             kcache: torch.Tensor, vcache: torch.Tensor, pdl: bool = False):
    """Decode-step RoPE of q (in place) and k, and the write of k, v into caches [B, nkv, T, D] at position *pos, which the
    caller keeps below T (cache slot and rotary angle both come from it)."""
    _need_cuda(q, k, v, cos, sin, pos, kcache, vcache)
    b, nkv, t, d = kcache.shape
    nq = q.numel() // (b * d)
    with torch.cuda.device(q.device):
        L.check(L.lib().wf_rope_kv_bf16(q.data_ptr(), k.data_ptr(), v.data_ptr(), cos.data_ptr(), sin.data_ptr(), pos.data_ptr(),
                                        kcache.data_ptr(), vcache.data_ptr(), b, nq, nkv, d, t, L.FLAG_PDL if pdl else 0, _stream()),
                "wf_rope_kv_bf16")


_attn_ws = {}


def attn_decode(q: torch.Tensor, kcache: torch.Tensor, vcache: torch.Tensor, pos: Optional[torch.Tensor], out: torch.Tensor,
                scale: Optional[float] = None, pdl: bool = False):
    """Decode-step attention over the bf16 KV cache: q [B, nq*D] (rotated), caches [B, nkv, T, D], `pos` a device
    scalar (positions 0..pos are attended to; None: all T), out [B, nq*D].  Grouped-query heads share one pass over
    their keys and values."""
    _need_cuda(q, kcache, vcache, pos, out)
    b, nkv, t, d = kcache.shape
    nq = q.numel() // (b * d)
    if q.dtype != torch.bfloat16 or kcache.dtype != torch.bfloat16 or not (kcache.is_contiguous() and vcache.is_contiguous()):
        raise ValueError("attn_decode needs contiguous bf16 tensors")
    lib = L.lib()
    nbytes = lib.wf_attn_decode_workspace_bytes(b, nq, nkv, d, t)
    ws = _attn_ws.get(q.device)
    if ws is None or ws.numel() < nbytes:
        ws = torch.zeros(max(nbytes, 1 << 16), dtype=torch.uint8, device=q.device)
        _attn_ws[q.device] = ws
    with torch.cuda.device(q.device):
        L.check(lib.wf_attn_decode_bf16(q.data_ptr(), kcache.data_ptr(), vcache.data_ptr(), _ptr(pos), out.data_ptr(), b, nq, nkv, d, t,
                                        float(scale if scale is not None else d ** -0.5), ws.data_ptr(), ws.numel(),
                                        L.FLAG_PDL if pdl else 0, _stream()), "wf_attn_decode_bf16")
    return out


def add_rmsnorm_quant_(h: torch.Tensor, delta: Optional[torch.Tensor], weight: torch.Tensor, q: torch.Tensor, q_scale: torch.Tensor,
                       eps: float, out: Optional[torch.Tensor] = None, quant_eps: float = 1e-5, pdl: bool = False):
    """h += delta (when given); the normalised row rmsnorm(h) * weight is quantized to int8 per token straight into
    `q` [M, K] / `q_scale` [M] (the bits of act_quant_i8 on the bf16 result) and written as bf16 into `out` when given."""
    _need_cuda(h, delta, weight, q, q_scale, out)
    m, k = h.shape
    with torch.cuda.device(h.device):
        L.check(L.lib().wf_add_rmsnorm_quant_bf16(h.data_ptr(), _ptr(delta), weight.data_ptr(), _ptr(out), q.data_ptr(), q_scale.data_ptr(),
                                                  m, k, float(eps), float(quant_eps), L.FLAG_PDL if pdl else 0, _stream()),
                "wf_add_rmsnorm_quant_bf16")
    return q, q_scale


def act_mul_quant(gate: torch.Tensor, up: torch.Tensor, q: torch.Tensor, q_scale: torch.Tensor, mode: str = "silu",
                  out: Optional[torch.Tensor] = None, quant_eps: float = 1e-5, pdl: bool = False):
    """act(gate) * up per token row [M, I], quantized to int8 per token into `q` / `q_scale` (and written as bf16 into
    `out` when given): the activation in front of down_proj with that projection's quantization."""
    _need_cuda(gate, up, q, q_scale, out)
    m, i = gate.shape
    with torch.cuda.device(gate.device):
        L.check(L.lib().wf_act_mul_quant_bf16(gate.data_ptr(), up.data_ptr(), _ptr(out), q.data_ptr(), q_scale.data_ptr(), m, i,
                                              0 if mode == "silu" else 1, float(quant_eps), L.FLAG_PDL if pdl else 0, _stream()),
                "wf_act_mul_quant_bf16")
    return q, q_scale


def linear_bf16(x: torch.Tensor, weight: torch.Tensor, out: Optional[torch.Tensor] = None, out_dtype: Optional[torch.dtype] = None,
                pdl: bool = False) -> torch.Tensor:
    """y = x @ weight.T for bf16 x [..., K] and weight [N, K] (fp32 accumulation on the tensor cores): the output head of
    the decoder, the one matrix the reference keeps in full precision.  `out` [..., N] of bf16 / f16 / f32 (default: bf16)."""
    _need_cuda(x, weight, out)
    k = x.shape[-1]
    x2 = x.reshape(-1, k)
    if x.dtype != torch.bfloat16 or weight.dtype != torch.bfloat16 or weight.dim() != 2 or weight.shape[1] != k:
        raise ValueError("linear_bf16 needs bf16 x [..., K] and weight [N, K]")
    if x2.stride(1) != 1:
        x2 = x2.contiguous()
    if weight.stride(1) != 1:
        raise ValueError("linear_bf16 needs weight rows with unit stride")
    m, n = x2.shape[0], weight.shape[0]
    if out is None:
        out = torch.empty(*x.shape[:-1], n, dtype=out_dtype or torch.bfloat16, device=x.device)
    y2 = out.view(-1, n) if out.dim() != 2 else out
    if y2.shape[0] != m or y2.stride(1) != 1 or out.dtype not in (torch.bfloat16, torch.float16, torch.float32):
        raise ValueError("linear_bf16: `out` must be [..., N] of bf16, f16 or f32 with unit inner stride")
    with torch.cuda.device(x.device):
        L.check(L.lib().wf_linear_bf16(x2.data_ptr(), x2.stride(0), weight.data_ptr(), weight.stride(0), y2.data_ptr(), _DT[out.dtype],
                                       y2.stride(0), m, n, k, L.FLAG_PDL if pdl else 0, _stream()), "wf_linear_bf16")
    return out


def act_mul(gate: torch.Tensor, up: torch.Tensor, out: torch.Tensor, mode: str = "silu", pdl: bool = False):
    """out = act(gate) * up (bf16); mode "silu" or "relu2"."""
    _need_cuda(gate, up, out)
    with torch.cuda.device(gate.device):
        L.check(L.lib().wf_act_mul_bf16(gate.data_ptr(), up.data_ptr(), out.data_ptr(), gate.numel(), 0 if mode == "silu" else 1,
                                        L.FLAG_PDL if pdl else 0, _stream()), "wf_act_mul_bf16")
    return out


def device_status() -> None:
    """Raises when a bounded wait inside a decode kernel ran out since the last check."""
    L.check(L.lib().wf_device_status(), "wf_device_status")


# --------------------------------------------------------------------------
# operator API of sgl_kernel.quantization.bitnet (same names, same argument meaning)
# --------------------------------------------------------------------------


def bitnet_gemv(packed_weights: torch.Tensor, activations: torch.Tensor, scale: float) -> torch.Tensor:
    """y = scale * (W @ x): packed I2_S weights [out, in/4] uint8, int8 activations [in] -> float32 [out]
    (sgl_kernel/quantization/bitnet.py:73-111)."""
    in_features = packed_weights.shape[1] * 4
    if in_features % QK_I2_S != 0:
        raise ValueError(f"bitnet_gemv: in_features ({in_features}) must be multiple of {QK_I2_S}")
    if activations.shape[0] != in_features:
        raise ValueError(f"bitnet_gemv: activations.shape[0] ({activations.shape[0]}) != in_features ({in_features})")
    return bitlinear(activations.reshape(1, -1), packed_weights, float(scale), layout=L.LAYOUT_I2S,
                     out_dtype=torch.float32, path="decode").reshape(-1)


def bitnet_gemm(packed_weights: torch.Tensor, activations: torch.Tensor, scale: float) -> torch.Tensor:
    """Y = scale * (X @ W^T): int8 activations [batch, in] -> float32 [batch, out]
    (sgl_kernel/quantization/bitnet.py:114-152)."""
    in_features = packed_weights.shape[1] * 4
    if in_features % QK_I2_S != 0:
        raise ValueError(f"bitnet_gemm: in_features ({in_features}) must be multiple of {QK_I2_S}")
    return bitlinear(activations, packed_weights, float(scale), layout=L.LAYOUT_I2S, out_dtype=torch.float32)


def quantize_activations_i8(activations: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """Per-tensor absmax int8 quantization; returns (int8 tensor, scale tensor [1])
    (sgl_kernel/quantization/bitnet.py:155-179)."""
    q, s = act_quant_i8(activations.float(), per_tensor=True)
    return q, s


def auto_tune_tiles(M: int, N: int, K: int) -> Tuple[int, int, int]:
    """Kept for API compatibility (sgl_kernel/quantization/bitnet.py:182-203); the GPU kernels
    pick their own tiling, the returned values are the reference's CPU heuristics."""
    return min(M, 64), min(N, 64), min(K, QK_I2_S * 2)
