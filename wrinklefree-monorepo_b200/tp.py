"""Tensor-parallel BitLinear: column-parallel (shard the output rows, no exchange) and
row-parallel (shard K, one all-reduce of the partial outputs).

Convention of the reference: q/k/v/gate/up are column-parallel, o/down row-parallel
(cheapertraining/_legacy/distributed/parallelism.py:148-193; sglang/srt/layers/linear.py:270-461
and :1224-1434), and the only collective on the path is the all-reduce after a row-parallel
projection (linear.py:1419-1420).

Weights are ternarized on the FULL matrix (one per-tensor absmean) and then sharded, so the
codes are the same at every tensor-parallel degree.  A row-parallel rank sees only its slice
of every token, so its activation scale is the absmax of that slice; each rank dequantizes its
partial sum with its own scale and the partial outputs are summed in `reduce_dtype`.

One process per GPU; the process group is passed in (NCCL on GPUs, gloo in the CPU tests).
"""
from __future__ import annotations

from typing import Callable, List, Optional, Tuple

import torch
import torch.distributed as dist
import torch.nn as nn

from . import _lib as L
from . import ops


class OneShotAllReduce:
    """Sum over the ranks of a process group for small CUDA tensors, by a kernel of this library that reads the
    partial tensors through peer memory (one process per GPU on one node).  It stands where the reference's
    row-parallel layers call the library all-reduce (linear.py:1419-1420); the sum runs in rank order in fp32, so
    all ranks obtain identical bits.  Tensors above `max_bytes`, of other dtypes or not 16-byte sized fall back to
    `dist.all_reduce`.  Set up collectively: every rank of `group` constructs it at the same point."""

    _DT = {torch.bfloat16: L.WF_BF16, torch.float16: L.WF_F16, torch.float32: L.WF_F32}

    def __init__(self, group=None, max_bytes: int = 1 << 20):
        import ctypes as C

        self.group = group
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        self.max_bytes = max_bytes
        self._ctx = None
        if self.world < 2 or self.world > 8 or not torch.cuda.is_available():
            return
        lib = L.lib()
        hb = lib.wf_ar_handle_bytes()
        handle = (C.c_ubyte * hb)()
        ctx = C.c_void_p()
        # Every step is collective: a rank whose set-up fails (no peer access, IPC not permitted) makes ALL ranks fall
        # back to the group's all_reduce, so the ranks never disagree about the path.
        ok = lib.wf_ar_init(self.world, self.rank, max_bytes, C.byref(ctx), handle) == 0
        gathered = [None] * self.world
        dist.all_gather_object(gathered, bytes(handle) if ok else None, group=group)
        ok = ok and all(h is not None for h in gathered)
        if ok:
            blob = b"".join(gathered)
            buf = (C.c_ubyte * len(blob)).from_buffer_copy(blob)
            ok = lib.wf_ar_connect(ctx, buf) == 0
        flag = torch.tensor([1 if ok else 0], device="cuda")
        dist.all_reduce(flag, op=dist.ReduceOp.MIN, group=group)  # also: every rank has mapped every buffer
        if int(flag.item()) == 1:
            self._ctx = ctx
        elif ctx.value:
            lib.wf_ar_destroy(ctx)

    def __call__(self, y: torch.Tensor, pdl: bool = False) -> torch.Tensor:
        """In-place sum of y over the ranks."""
        nbytes = y.numel() * y.element_size()
        if (self._ctx is None or y.dtype not in self._DT or not y.is_contiguous() or nbytes > self.max_bytes or nbytes % 16
                or y.data_ptr() % 16):
            if self.world > 1:
                dist.all_reduce(y, op=dist.ReduceOp.SUM, group=self.group)
            return y
        with torch.cuda.device(y.device):
            L.check(L.lib().wf_ar_allreduce(self._ctx, y.data_ptr(), y.data_ptr(), y.numel(), self._DT[y.dtype],
                                            L.FLAG_PDL if pdl else 0, torch.cuda.current_stream().cuda_stream), "wf_ar_allreduce")
        return y

    def xchg_ptr(self):
        """Device pointer of this exchange's descriptor, for `DecodeGroup(..., xchg=ptr)`: the row-parallel projection
        then pushes its partial output to every rank itself; `reduce_add_rmsnorm_` is the matching consumer.  None when
        the peer-memory path is not available."""
        import ctypes as C

        if self._ctx is None:
            return None
        p = C.c_void_p()
        L.check(L.lib().wf_ar_xchg(self._ctx, C.byref(p)), "wf_ar_xchg")
        return p.value

    def reduce_add_rmsnorm_(self, h: torch.Tensor, weight: torch.Tensor, y: Optional[torch.Tensor], eps: float, pdl: bool = False,
                            q: Optional[torch.Tensor] = None, q_scale: Optional[torch.Tensor] = None, quant_eps: float = 1e-5):
        """Consumer of a fused exchange, on every rank after the pushing launch: h += sum over the ranks of the pushed
        partial outputs (fp32 in rank order, rounded to bf16: the bits of the stand-alone all-reduce), y = rmsnorm(h) * weight.
        With `q` / `q_scale` the normalised row is also quantized to int8 per token (the bits of act_quant_i8); y may then be None."""
        if self._ctx is None:
            raise RuntimeError("the peer-memory exchange is not available on this group")
        m, k = h.shape
        ptr = lambda t: None if t is None else t.data_ptr()
        with torch.cuda.device(h.device):
            L.check(L.lib().wf_ar_reduce_add_rmsnorm_quant(self._ctx, h.data_ptr(), weight.data_ptr(), ptr(y), ptr(q), ptr(q_scale), m, k,
                                                           float(eps), float(quant_eps), L.FLAG_PDL if pdl else 0,
                                                           torch.cuda.current_stream().cuda_stream), "wf_ar_reduce_add_rmsnorm")
        return y if q is None else (q, q_scale)

    def status(self) -> None:
        """Raises if a bounded wait for a peer ran out since the last call."""
        import ctypes as C

        if self._ctx is None:
            return
        v = C.c_int(0)
        L.check(L.lib().wf_ar_status(self._ctx, C.byref(v)), "wf_ar_status")
        if v.value:
            raise RuntimeError("one-shot all-reduce: a wait for a peer ran out (a rank did not take part)")


    def resync(self) -> None:
        """Collective, after `status()` raised on any rank: puts every rank on one common step and clears the status,
        so that the next all-reduce runs normally.  (A rank that sat out a call is behind the others by one step; the
        flags of the ranks that waited in vain are ahead of it.)"""
        import ctypes as C

        if self._ctx is None:
            return
        lib = L.lib()
        v = C.c_uint(0)
        L.check(lib.wf_ar_step(self._ctx, C.byref(v)), "wf_ar_step")
        t = torch.tensor([v.value], dtype=torch.int64, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX, group=self.group)  # also: nobody is inside an all-reduce any more
        L.check(lib.wf_ar_set_step(self._ctx, int(t.item()) + 2), "wf_ar_set_step")
        dist.barrier(group=self.group)  # nobody launches before every rank has set the step


def shard_bounds(total: int, parts: int, align: int) -> List[Tuple[int, int]]:
    """Splits [0, total) into `parts` contiguous ranges whose sizes are multiples of `align`
    and differ by at most one unit (the first ranges take the larger share)."""
    if total % align:
        raise ValueError(f"{total} is not a multiple of {align}")
    units = total // align
    if units < parts:
        raise ValueError(f"cannot split {units} units of {align} over {parts} ranks")
    base, extra = divmod(units, parts)
    out, lo = [], 0
    for r in range(parts):
        hi = lo + (base + (1 if r < extra else 0)) * align
        out.append((lo, hi))
        lo = hi
    return out


def shard_codes_rows(codes: torch.Tensor, lo: int, hi: int) -> torch.Tensor:
    """Rows [lo, hi) of packed weights [N, K/4] (any row-major layout)."""
    return codes[lo:hi].contiguous()


def shard_codes_k(codes: torch.Tensor, k_lo: int, k_hi: int, layout: int = L.LAYOUT_WF16) -> torch.Tensor:
    """Input features [k_lo, k_hi) of packed weights [N, K/4].  A slice of bytes is a slice of K when the
    bounds fall on the layout's block: 16 weights for WF16 (64 for the kernels' vector loads), 128 for I2_S
    (the reference narrows the byte tensor the same way, linear.py:1309-1368)."""
    block = 128 if layout == L.LAYOUT_I2S else 64
    if k_lo % block or k_hi % block:
        raise ValueError(f"K shard [{k_lo}, {k_hi}) must fall on multiples of {block}")
    return codes[:, k_lo // 4 : k_hi // 4].contiguous()


class _ParallelBase(nn.Module):
    def __init__(self, group, linear_fn: Optional[Callable]):
        super().__init__()
        self.group = group
        self.tp_size = dist.get_world_size(group) if (group is not None or dist.is_initialized()) else 1
        self.tp_rank = dist.get_rank(group) if (group is not None or dist.is_initialized()) else 0
        self._linear = linear_fn or ops.bitlinear


class ColumnParallelBitLinear(_ParallelBase):
    """y_local = BitLinear(x)[..., rows of this rank]; optional all-gather of the outputs."""

    def __init__(self, codes_full: torch.Tensor, w_scale, in_features: int, out_features: int, group=None,
                 bias: Optional[torch.Tensor] = None, gather_output: bool = False, layout: int = L.LAYOUT_WF16,
                 row_align: int = 16, linear_fn: Optional[Callable] = None):
        super().__init__(group, linear_fn)
        self.in_features, self.out_features, self.layout, self.gather_output = in_features, out_features, layout, gather_output
        self.bounds = shard_bounds(out_features, self.tp_size, row_align)
        lo, hi = self.bounds[self.tp_rank]
        self.register_buffer("codes", shard_codes_rows(codes_full, lo, hi))
        self.w_scale = w_scale
        self.register_buffer("bias", bias[lo:hi].contiguous() if bias is not None else None)

    def forward(self, x: torch.Tensor, **kw) -> torch.Tensor:
        y = self._linear(x, self.codes, self.w_scale, bias=self.bias, layout=self.layout, **kw)
        if not self.gather_output or self.tp_size == 1:
            return y
        sizes = [hi - lo for lo, hi in self.bounds]
        parts = [torch.empty(*y.shape[:-1], s, dtype=y.dtype, device=y.device) for s in sizes]
        dist.all_gather(parts, y.contiguous(), group=self.group)
        return torch.cat(parts, dim=-1)


class RowParallelBitLinear(_ParallelBase):
    """y = sum over ranks of BitLinear_k-slice(x_local); one all-reduce, bias added on rank 0 only
    (as linear.py:1412-1414 does)."""

    def __init__(self, codes_full: torch.Tensor, w_scale, in_features: int, out_features: int, group=None,
                 bias: Optional[torch.Tensor] = None, input_is_parallel: bool = True, layout: int = L.LAYOUT_WF16,
                 reduce_dtype: Optional[torch.dtype] = None, linear_fn: Optional[Callable] = None,
                 all_reduce: Optional[Callable] = None):
        super().__init__(group, linear_fn)
        self.all_reduce = all_reduce  # e.g. a OneShotAllReduce of the same group; default: dist.all_reduce
        self.in_features, self.out_features, self.layout = in_features, out_features, layout
        self.input_is_parallel, self.reduce_dtype = input_is_parallel, reduce_dtype
        self.bounds = shard_bounds(in_features, self.tp_size, 128 if layout == L.LAYOUT_I2S else 64)
        lo, hi = self.bounds[self.tp_rank]
        self.register_buffer("codes", shard_codes_k(codes_full, lo, hi, layout))
        self.w_scale = w_scale
        self.register_buffer("bias", bias if (bias is not None and self.tp_rank == 0) else None)

    def forward(self, x: torch.Tensor, **kw) -> torch.Tensor:
        if not self.input_is_parallel:
            lo, hi = self.bounds[self.tp_rank]
            x = x[..., lo:hi]
        out_dtype = kw.pop("out_dtype", None) or (torch.float32 if x.dtype == torch.int8 else x.dtype)
        red = self.reduce_dtype or out_dtype
        y = self._linear(x, self.codes, self.w_scale, bias=self.bias, layout=self.layout, out_dtype=red, **kw)
        if self.tp_size > 1:
            if self.all_reduce is not None:
                self.all_reduce(y)
            else:
                dist.all_reduce(y, op=dist.ReduceOp.SUM, group=self.group)
        return y if red == out_dtype else y.to(out_dtype)


def column_parallel_from_weight(weight: torch.Tensor, group=None, mode: torch.dtype = torch.float32, **kw):
    """Ternarize the full latent weight [N, K] on the GPU, keep this rank's rows."""
    codes, scale = ops.pack_ternary(weight, mode=mode)
    return ColumnParallelBitLinear(codes, scale, weight.shape[1], weight.shape[0], group=group, **kw)


def row_parallel_from_weight(weight: torch.Tensor, group=None, mode: torch.dtype = torch.float32, **kw):
    """Ternarize the full latent weight [N, K] on the GPU, keep this rank's slice of K."""
    codes, scale = ops.pack_ternary(weight, mode=mode)
    return RowParallelBitLinear(codes, scale, weight.shape[1], weight.shape[0], group=group, **kw)
