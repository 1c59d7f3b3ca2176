"""A minimal LLaMA-style ternary decoder used to measure decode tokens/s on the BitLinear kernels.

Skeleton after the reference's model (wrinklefree/models/attention.py:126-218, ffn.py:43-87, llama.py:81-238):
RMSNorm -> q/k/v BitLinear -> RoPE -> GQA attention -> o BitLinear -> residual -> RMSNorm -> gate/up BitLinear ->
act(gate) * up -> down BitLinear -> residual; bf16 embedding and lm_head.  Unlike the reference it keeps a bf16
KV cache, launches q/k/v and gate/up as one grouped kernel each, and replays the whole decode step as a CUDA
graph.  With `subln=True` and weights loaded under the reference's parameter names it computes the reference
model (BitNetLlama) itself.  In the decode step the norms, RoPE + cache write, attention over the cache and the gate
activation are kernels of this library as well; the prompt pass uses stock torch operators around the projections.

Tensor parallel: heads and the MLP width are split over the ranks of a process group; q/k/v/gate/up are
column-parallel, o/down row-parallel with one all-reduce each (the reference's plan); the output head is sharded by
vocabulary rows and the greedy token comes from one all-gather of per-rank (maximum, index) pairs.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Optional

import torch
import torch.distributed as dist
import torch.nn.functional as F

from . import ops
from . import tp as tpmod


@dataclass
class DecoderConfig:
    layers: int
    hidden: int
    n_q: int
    n_kv: int
    head_dim: int
    intermediate: int
    vocab: int
    rope_theta: float = 1e5
    act: str = "silu"  # "silu" (SwiGLU) or "relu2" (the reference's SmolLM2 preset)
    eps: float = 1e-5  # RMSNorm epsilon (the reference's rms_norm_eps defaults to 1e-6)
    subln: bool = False  # sub-layer norms in front of o_proj and down_proj (wrinklefree/models/attention.py:213, ffn.py:84)
    subln_eps: float = 1e-6


SMOLLM2_135M = DecoderConfig(layers=30, hidden=576, n_q=9, n_kv=3, head_dim=64, intermediate=1536, vocab=49152, rope_theta=1e5)
LLAMA3_8B = DecoderConfig(layers=32, hidden=4096, n_q=32, n_kv=8, head_dim=128, intermediate=14336, vocab=128256, rope_theta=5e5)


def _rms_norm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    v = x.float()
    return (v * torch.rsqrt(v.pow(2).mean(-1, keepdim=True) + eps)).to(x.dtype) * w


def _rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """x [B, H, T, D]; cos/sin [T, D/2] (or broadcastable)."""
    x1, x2 = x[..., : x.shape[-1] // 2], x[..., x.shape[-1] // 2 :]
    return torch.cat([x1 * cos - x2 * sin, x2 * cos + x1 * sin], dim=-1).to(x.dtype)


def _causal_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor) -> torch.Tensor:
    """Prompt attention, q [B, Hq, S, D], k/v [B, Hkv, S, D].  Low-precision inputs use the fused library kernel; fp32
    inputs are evaluated with plain fp32 matrix products and an fp32 softmax, as the reference's attention does
    (attention.py:189-208) - the fused kernels round fp32 operands to TF32."""
    if q.dtype != torch.float32:
        return F.scaled_dot_product_attention(q, k, v, is_causal=True, enable_gqa=True)
    rep = q.shape[1] // k.shape[1]
    k, v = k.repeat_interleave(rep, dim=1), v.repeat_interleave(rep, dim=1)
    S = q.shape[2]
    scores = torch.matmul(q, k.transpose(-2, -1)) * (1.0 / math.sqrt(q.shape[-1]))
    scores = scores + torch.full((S, S), float("-inf"), device=q.device).triu(1)
    return torch.matmul(torch.softmax(scores, dim=-1), v)


class TernaryDecoder:
    """Random-initialised ternary decoder (weights N(0, 0.02), ternarized on the GPU)."""

    def __init__(self, cfg: DecoderConfig, batch: int, max_ctx: int, device, group=None, seed: int = 0,
                 dtype: torch.dtype = torch.bfloat16, weights: Optional[dict] = None, pack_mode: torch.dtype = torch.float32,
                 fuse: Optional[bool] = None, prefetch: bool = False, fuse_exchange: Optional[bool] = None):
        """`weights`: optional fp32 state dict under the reference model's parameter names (BitNetLlama,
        wrinklefree/models/llama.py:13-59); without it the weights are drawn from N(0, 0.02) with `seed`.
        `pack_mode`: arithmetic of the ternarization (torch.float32, or the input dtype for the cast-first rule of
        BitLinear.forward).  `fuse`: True runs the decode step of small batches with the fused input modes of the
        grouped kernel (six launches per layer instead of ten); measured on B200 the separate norm / activation kernels,
        which overlap the projections' weight streaming through programmatic launches, are faster, so it is off by
        default.  `fuse_exchange` (tensor parallel, up to 8 sequences, bf16): the row-parallel projections push their partial
        outputs to every rank inside their own launch and the residual add + RMSNorm that follows sums them (default: from two
        sequences on; True / False force it)."""
        self._fuse_opt = fuse
        # tensor parallel, few tokens: False keeps the exchange after o_proj / down_proj a kernel of its own
        self._xchg_opt = fuse_exchange
        # decode step: every projection group asks L2 for the following launches' weights.  Measured on B200 at batch 1
        # (8B shape) this made the step slower (2.05 -> 2.25 ms: the prefetch competes with the running launch's own
        # stream), so it is off by default.
        self.prefetch = prefetch
        self.cfg, self.B, self.T, self.dev, self.dtype, self.group = cfg, batch, max_ctx, device, dtype, group
        self._oneshot = None  # peer-memory all-reduce for the row-parallel projections (set up at the first step)
        self.tp = dist.get_world_size(group) if (group is not None or dist.is_initialized()) else 1
        self.rank = dist.get_rank(group) if (group is not None or dist.is_initialized()) else 0
        if cfg.n_kv % self.tp or cfg.n_q % self.tp:
            raise ValueError("heads must divide over the tensor-parallel ranks")
        if cfg.subln and self.tp > 1:
            raise NotImplementedError("sub-layer norms over a sharded width need one more exchange; not built for tp > 1")
        self.nq, self.nkv = cfg.n_q // self.tp, cfg.n_kv // self.tp
        self.i_lo, self.i_hi = tpmod.shard_bounds(cfg.intermediate, self.tp, 64)[self.rank]
        d, h = cfg.head_dim, cfg.hidden
        gen = torch.Generator(device=device).manual_seed(seed)  # same seed on every rank: same full matrices
        # The reference rotates interleaved pairs (2i, 2i+1) of a head (attention.py:41-64); the kernels here rotate
        # the pairs (i, i + d/2).  Scores are invariant under one permutation of q and k inside every head, so loaded
        # q/k weights are permuted once: new row i = old row 2i, new row i + d/2 = old row 2i + 1.
        perm = torch.cat([torch.arange(0, d, 2), torch.arange(1, d, 2)])

        def given(name, n, k, heads=0):
            w = weights[name].to(device=device, dtype=torch.float32)
            if tuple(w.shape) != (n, k):
                raise ValueError(f"{name}: expected {(n, k)}, got {tuple(w.shape)}")
            if heads:
                w = w.view(heads, d, k)[:, perm.to(device)].reshape(n, k)
            return w

        def ternary(n, k, name=None, heads=0):
            if weights is not None:
                w = given(name, n, k, heads)
            else:
                w = torch.randn(n, k, generator=gen, device=device, dtype=torch.float32) * 0.02
            c, s = ops.pack_ternary(w, mode=pack_mode, eps=1e-5)
            return c, s

        def vec(name, n):
            if weights is not None and name in weights:
                return weights[name].to(device=device, dtype=dtype).contiguous()
            return torch.ones(n, dtype=dtype, device=device)

        self.layers = []
        for li in range(cfg.layers):
            L = {}
            pre = f"transformer.layers.{li}."
            cq, sq = ternary(cfg.n_q * d, h, pre + "self_attn.q_proj.weight", cfg.n_q)
            ck, sk = ternary(cfg.n_kv * d, h, pre + "self_attn.k_proj.weight", cfg.n_kv)
            cv, sv = ternary(cfg.n_kv * d, h, pre + "self_attn.v_proj.weight")
            co, so = ternary(h, cfg.n_q * d, pre + "self_attn.o_proj.weight")
            cg, sg = ternary(cfg.intermediate, h, pre + "mlp.gate_proj.weight")
            cu, su = ternary(cfg.intermediate, h, pre + "mlp.up_proj.weight")
            cd, sd = ternary(h, cfg.intermediate, pre + "mlp.down_proj.weight")
            r = self.rank
            L["q"] = (tpmod.shard_codes_rows(cq, r * self.nq * d, (r + 1) * self.nq * d), sq)
            L["k"] = (tpmod.shard_codes_rows(ck, r * self.nkv * d, (r + 1) * self.nkv * d), sk)
            L["v"] = (tpmod.shard_codes_rows(cv, r * self.nkv * d, (r + 1) * self.nkv * d), sv)
            L["o"] = (tpmod.shard_codes_k(co, r * self.nq * d, (r + 1) * self.nq * d), so)
            L["gate"] = (tpmod.shard_codes_rows(cg, self.i_lo, self.i_hi), sg)
            L["up"] = (tpmod.shard_codes_rows(cu, self.i_lo, self.i_hi), su)
            L["down"] = (tpmod.shard_codes_k(cd, self.i_lo, self.i_hi), sd)
            L["n1"] = vec(pre + "input_layernorm.weight", h)
            L["n2"] = vec(pre + "post_attention_layernorm.weight", h)
            if cfg.subln:
                L["sa"] = vec(pre + "self_attn.subln.weight", cfg.n_q * d)
                L["sf"] = vec(pre + "mlp.subln.weight", cfg.intermediate)
            L["kc"] = torch.zeros(batch, self.nkv, max_ctx, d, dtype=dtype, device=device)
            L["vc"] = torch.zeros(batch, self.nkv, max_ctx, d, dtype=dtype, device=device)
            self.layers.append(L)
        if weights is not None:
            self.embed = weights["embed_tokens.weight"].to(device=device, dtype=dtype)
            self.lm_head = weights["lm_head.weight"].to(device=device, dtype=dtype) if "lm_head.weight" in weights else self.embed
        else:
            self.embed = (torch.randn(cfg.vocab, h, generator=gen, device=device, dtype=torch.float32) * 0.02).to(dtype)
            self.lm_head = (torch.randn(cfg.vocab, h, generator=gen, device=device, dtype=torch.float32) * 0.02).to(dtype)
        self.norm_f = vec("transformer.norm.weight", h)
        # tensor parallel: the output head is sharded by vocabulary rows; every rank scores its rows, and the greedy token
        # is the best of the per-rank (maximum, index) pairs - one small all-gather per step instead of streaming the
        # whole head on every rank
        self.v_lo, self.v_hi = (0, cfg.vocab)
        if self.tp > 1:
            self.v_lo, self.v_hi = tpmod.shard_bounds(cfg.vocab, self.tp, 1)[self.rank]
            self.lm_head = self.lm_head[self.v_lo:self.v_hi].contiguous()
            self._cand = torch.empty(self.tp, 2, batch, dtype=torch.float32, device=device)
        inv = 1.0 / (cfg.rope_theta ** (torch.arange(0, d, 2, device=device, dtype=torch.float32) / d))
        ang = torch.arange(max_ctx, device=device, dtype=torch.float32)[:, None] * inv[None, :]
        self.cos, self.sin = ang.cos(), ang.sin()
        # static decode-step buffers (graph inputs / outputs)
        self.tok = torch.zeros(batch, dtype=torch.long, device=device)
        self.pos = torch.zeros((), dtype=torch.long, device=device)
        self._pos_host = 0  # host mirror of pos for the bound check of decode()
        self.masked, self.attention = True, "kernel"
        self._step_bufs()
        self.graph: Optional[torch.cuda.CUDAGraph] = None
        self.next_tok = torch.zeros(batch, dtype=torch.long, device=device)

    # ------------------------------------------------------------------ decode step buffers and groups
    def _step_bufs(self):
        """Static buffers and launch groups of the decode step.  Small batches (the projections on the fused
        quantize-and-contract kernel) use the fused input modes: the residual add + RMSNorm runs inside the q/k/v and
        gate/up launches and the gate activation inside the down launch, six launches per layer.  The residual stream
        alternates between two buffers (a fused launch reads one and writes the other)."""
        cfg, B, d, dev, dt = self.cfg, self.B, self.cfg.head_dim, self.dev, self.dtype
        self.big = B >= 16 and cfg.hidden >= 2048  # projections on the tensor-core contraction for few tokens
        self.fused = dt == torch.bfloat16 and not self.big and not cfg.subln and cfg.hidden % 8 == 0 and self._fuse_opt is True
        self.h = torch.empty(B, cfg.hidden, dtype=dt, device=dev)
        self.h2 = torch.empty(B, cfg.hidden, dtype=dt, device=dev)
        self.xf = torch.empty(B, cfg.hidden, dtype=dt, device=dev)
        self.head_out = torch.empty(B, self.lm_head.shape[0], dtype=dt, device=dev) if dt == torch.bfloat16 else None
        # Tensor parallel, few tokens: the exchange after o_proj / down_proj is fused into those launches (they push their
        # partial outputs to every rank) and into the residual add + RMSNorm that follows (it sums what was pushed).
        self.fuse_exchange = False
        if self.tp > 1 and self._xchg_opt is not False:
            if self._oneshot is None:
                self._oneshot = tpmod.OneShotAllReduce(self.group, max_bytes=64 << 10)  # measured: NCCL is faster from 256 KB on
            # measured on two B200s, 8B shape: 2 % faster than the exchange as a kernel of its own at 4 sequences, 2-5 %
            # slower at 1 (every CTA of the projection ends with its push): on from two sequences unless asked for
            wanted = self._xchg_opt is True or B >= 2
            self.fuse_exchange = (wanted and dt == torch.bfloat16 and not self.big and not self.fused and cfg.hidden % 8 == 0
                                  and cfg.hidden <= 16384 and B * cfg.hidden * 2 <= self._oneshot.max_bytes
                                  and self._oneshot.xchg_ptr() is not None)
        # The norms in front of q/k/v and gate/up, and the activation (or its sub-norm) in front of down, quantize their
        # result to int8 themselves where the projection would otherwise run a quantization kernel of its own.
        i_loc = self.i_hi - self.i_lo
        self.qnorm = (dt == torch.bfloat16 and not self.fused and cfg.hidden % 8 == 0 and cfg.hidden <= 16384
                      and ops._prequant(B, cfg.hidden, 2))
        self.qact = (dt == torch.bfloat16 and not self.fused and i_loc % 8 == 0 and i_loc <= 16384 and ops._prequant(B, i_loc, 1))
        mode = "silu" if cfg.act == "silu" else "relu2"
        prev_down = None
        for li, L in enumerate(self.layers):
            L["xn"] = torch.empty(B, cfg.hidden, dtype=dt, device=dev)
            L["qkv"] = [torch.empty(B, self.nq * d, dtype=dt, device=dev), torch.empty(B, self.nkv * d, dtype=dt, device=dev),
                        torch.empty(B, self.nkv * d, dtype=dt, device=dev)]
            L["hn"] = torch.empty(B, cfg.hidden, dtype=dt, device=dev)
            L["gu"] = [torch.empty(B, self.i_hi - self.i_lo, dtype=dt, device=dev) for _ in range(2)]
            L["act"] = torch.empty(B, self.i_hi - self.i_lo, dtype=dt, device=dev)
            L["attn"] = torch.empty(B, self.nq * d, dtype=dt, device=dev)
            if cfg.subln:
                L["an"] = torch.empty(B, self.nq * d, dtype=dt, device=dev)
                L["actn"] = torch.empty(B, self.i_hi - self.i_lo, dtype=dt, device=dev)
            L["ob"] = torch.empty(B, cfg.hidden, dtype=dt, device=dev)
            L["db"] = torch.empty(B, cfg.hidden, dtype=dt, device=dev)
            if self.qnorm:
                for nm in ("xn", "hn"):
                    L[nm + "_q"] = torch.empty(B, cfg.hidden, dtype=torch.int8, device=dev)
                    L[nm + "_s"] = torch.empty(B, dtype=torch.float32, device=dev)
            if self.qact:
                L["act_q"] = torch.empty(B, i_loc, dtype=torch.int8, device=dev)
                L["act_s"] = torch.empty(B, dtype=torch.float32, device=dev)
            if self.fused:
                # q/k/v: rmsnorm(h + previous down output) -> h2;  gate/up: rmsnorm(h2 + o output) -> h
                first = dict(x_mode="norm", x2=prev_down, norm_w=L["n1"], norm_eps=cfg.eps)
                L["g_qkv"] = ops.DecodeGroup([dict(x=self.h, codes=L[n][0], w_scale=L[n][1], out=o, h_out=self.h2 if n == "q" else None, **first)
                                              for n, o in zip(("q", "k", "v"), L["qkv"])])
                L["g_o"] = ops.DecodeGroup([dict(x=L["attn"], codes=L["o"][0], w_scale=L["o"][1], out=L["ob"])])
                second = dict(x_mode="norm", x2=L["ob"], norm_w=L["n2"], norm_eps=cfg.eps)
                L["g_gu"] = ops.DecodeGroup([dict(x=self.h2, codes=L[n][0], w_scale=L[n][1], out=o, h_out=self.h if n == "gate" else None, **second)
                                             for n, o in zip(("gate", "up"), L["gu"])])
                L["g_down"] = ops.DecodeGroup([dict(x=L["gu"][0], x2=L["gu"][1], x_mode=mode, codes=L["down"][0], w_scale=L["down"][1], out=L["db"])])
                prev_down = L["db"]
            else:
                # every group asks L2 for the weights of the launches that follow it, so that their HBM transfer overlaps
                # this chain of short launches: q/k/v -> o, gate, up;  gate/up -> down, the next layer's q
                nxt = self.layers[li + 1] if li + 1 < len(self.layers) else None
                pf1 = {"q": L["o"][0], "k": L["gate"][0], "v": L["up"][0]} if self.prefetch else {}
                pf2 = {"gate": L["down"][0], "up": nxt["q"][0] if nxt else None} if self.prefetch else {}
                xin = dict(x=L["xn_q"], x_scale=L["xn_s"]) if self.qnorm else dict(x=L["xn"])
                hin = dict(x=L["hn_q"], x_scale=L["hn_s"]) if self.qnorm else dict(x=L["hn"])
                L["g_qkv"] = ops.DecodeGroup([dict(codes=L[n][0], w_scale=L[n][1], out=o, prefetch=pf1.get(n), **xin)
                                              for n, o in zip(("q", "k", "v"), L["qkv"])])
                L["g_gu"] = ops.DecodeGroup([dict(codes=L[n][0], w_scale=L[n][1], out=o, prefetch=pf2.get(n), **hin)
                                             for n, o in zip(("gate", "up"), L["gu"])])
                if self.fuse_exchange:
                    xp = self._oneshot.xchg_ptr()
                    L["g_o"] = ops.DecodeGroup([dict(x=L["an"] if cfg.subln else L["attn"], codes=L["o"][0], w_scale=L["o"][1], out=L["ob"], xchg=xp)])
                    din = dict(x=L["act_q"], x_scale=L["act_s"]) if self.qact else dict(x=L["actn"] if cfg.subln else L["act"])
                    L["g_down"] = ops.DecodeGroup([dict(codes=L["down"][0], w_scale=L["down"][1], out=L["db"], xchg=xp, **din)])

    def _act(self, g, u):
        return (F.silu(g) if self.cfg.act == "silu" else F.relu(g).pow(2)) * u

    def _allreduce(self, y):
        if self.tp > 1:
            if self._oneshot is None:
                self._oneshot = tpmod.OneShotAllReduce(self.group, max_bytes=64 << 10)  # measured: NCCL is faster from 256 KB on
            self._oneshot(y, pdl=True)
        return y

    def _decode_step(self):
        """One token per sequence: reads self.tok / self.pos, writes self.next_tok; advances self.pos.
        Per layer: add+RMSNorm, q/k/v group, RoPE+cache write, attention, o, add+RMSNorm, gate/up group,
        activation*up, down -- ten launches, chained with programmatic dependencies: every kernel of this library
        starts while its predecessor drains (the projections stream their first weights meanwhile) and waits for it
        before it reads an activation."""
        cfg, B, d = self.cfg, self.B, self.cfg.head_dim
        self.h.copy_(self.embed[self.tok])  # residual stream [B, hidden]
        if self.fused:
            return self._decode_step_fused()
        valid = None
        if self.masked and self.attention == "library":
            valid = (torch.arange(self.T, device=self.dev) <= self.pos).view(1, 1, 1, self.T)
        delta = None
        fx = self.fuse_exchange
        for L in self.layers:
            if fx and delta is not None:  # the previous layer's down projection has pushed its partial outputs
                if self.qnorm:
                    self._oneshot.reduce_add_rmsnorm_(self.h, L["n1"], None, cfg.eps, pdl=True, q=L["xn_q"], q_scale=L["xn_s"])
                else:
                    self._oneshot.reduce_add_rmsnorm_(self.h, L["n1"], L["xn"], cfg.eps, pdl=True)
            elif self.qnorm:
                ops.add_rmsnorm_quant_(self.h, delta, L["n1"], L["xn_q"], L["xn_s"], cfg.eps, pdl=True)
            else:
                ops.add_rmsnorm_(self.h, delta, L["n1"], L["xn"], cfg.eps, pdl=True)
            q, k, v = L["g_qkv"].run(pdl=True)
            ops.rope_kv_(q, k, v, self.cos, self.sin, self.pos, L["kc"], L["vc"], pdl=True)
            if self.attention == "library":  # the framework's fused kernel, kept as a comparison for the benchmark
                a = F.scaled_dot_product_attention(q.view(B, self.nq, 1, d), L["kc"], L["vc"], attn_mask=valid, enable_gqa=True)
            else:
                a = ops.attn_decode(q, L["kc"], L["vc"], self.pos if self.masked else None, L["attn"], pdl=True)
            # from 16 sequences on the single projections of a wide model run on the tensor-core contraction for few
            # tokens (measured: 14 vs 20 us for 4096 x 4096 at 32 tokens; narrow layers stay faster on the decode kernel)
            big = self.big
            path = "prefill" if big else "decode"
            a = a.reshape(B, self.nq * d)
            if cfg.subln:
                a = ops.add_rmsnorm_(a, None, L["sa"], L["an"], cfg.subln_eps, pdl=True)
            if fx:
                if a.data_ptr() != L["g_o"].x_ptr:
                    L["attn"].copy_(a)  # the comparison attention writes its own tensor
                L["g_o"].run(pdl=True)
                if self.qnorm:
                    self._oneshot.reduce_add_rmsnorm_(self.h, L["n2"], None, cfg.eps, pdl=True, q=L["hn_q"], q_scale=L["hn_s"])
                else:
                    self._oneshot.reduce_add_rmsnorm_(self.h, L["n2"], L["hn"], cfg.eps, pdl=True)
            else:
                o = self._allreduce(ops.bitlinear(a, L["o"][0], L["o"][1], out=L["ob"], path=path, pdl=True))
                if self.qnorm:
                    ops.add_rmsnorm_quant_(self.h, o, L["n2"], L["hn_q"], L["hn_s"], cfg.eps, pdl=True)
                else:
                    ops.add_rmsnorm_(self.h, o, L["n2"], L["hn"], cfg.eps, pdl=True)
            if big:
                # one quantization for gate and up
                hq, hs = (L["hn_q"], L["hn_s"]) if self.qnorm else ops.act_quant_i8(L["hn"], eps=1e-5)
                g, u = (ops.bitlinear(hq, L[n][0], L[n][1], x_scale=hs, out=o_, path="prefill")
                        for n, o_ in zip(("gate", "up"), L["gu"]))
            else:
                g, u = L["g_gu"].run(pdl=True)
            act_s = None
            if cfg.subln:
                act = ops.act_mul(g, u, L["act"], self.cfg.act, pdl=True)
                if self.qact:
                    act, act_s = ops.add_rmsnorm_quant_(act, None, L["sf"], L["act_q"], L["act_s"], cfg.subln_eps, pdl=True)
                else:
                    act = ops.add_rmsnorm_(act, None, L["sf"], L["actn"], cfg.subln_eps, pdl=True)
            elif self.qact:
                act, act_s = ops.act_mul_quant(g, u, L["act_q"], L["act_s"], self.cfg.act, pdl=True)
            else:
                act = ops.act_mul(g, u, L["act"], self.cfg.act, pdl=True)
            if fx:
                delta = L["g_down"].run(pdl=True)[0]
            else:
                delta = self._allreduce(ops.bitlinear(act, L["down"][0], L["down"][1], x_scale=act_s, out=L["db"], path=path, pdl=True))
        if fx:
            self._oneshot.reduce_add_rmsnorm_(self.h, self.norm_f, self.xf, cfg.eps, pdl=True)
        else:
            ops.add_rmsnorm_(self.h, delta, self.norm_f, self.xf, cfg.eps, pdl=True)
        self._greedy(self._head(self.xf, self.head_out, pdl=True))
        self.pos.add_(1)

    def _head(self, x, out=None, pdl=False):
        """This rank's rows of the output head: a kernel of this library for bf16, the framework's matmul for the fp32
        model that the parity tests hold against the reference."""
        if x.dtype == torch.bfloat16 and self.lm_head.dtype == torch.bfloat16:
            return ops.linear_bf16(x, self.lm_head, out=out, pdl=pdl)
        return x @ self.lm_head.t()

    def _greedy(self, logits):
        """next_tok = argmax over the vocabulary; `logits` are this rank's rows of the head."""
        self.logits = logits
        if self.tp == 1:
            self.next_tok.copy_(logits.argmax(-1))
            return
        mx, idx = logits.float().max(-1)
        mine = torch.stack([mx, (idx + self.v_lo).float()])  # vocabulary indices are exact in fp32 (< 2^24)
        dist.all_gather_into_tensor(self._cand.view(-1), mine.view(-1), group=self.group)
        best = self._cand[:, 0].argmax(0)  # [B]: the rank that holds the maximum (the lowest rank on ties)
        self.next_tok.copy_(self._cand[:, 1].gather(0, best.unsqueeze(0)).squeeze(0).long())

    def _decode_step_fused(self):
        """Six launches per layer: q/k/v (residual add + RMSNorm + quantization fused in), RoPE + cache write, attention,
        o, gate/up (residual add + RMSNorm fused in), down (gate activation fused in); with tensor parallelism the two
        row-parallel outputs are summed over the ranks in between."""
        cfg = self.cfg
        for L in self.layers:
            q, k, v = L["g_qkv"].run(pdl=True)
            ops.rope_kv_(q, k, v, self.cos, self.sin, self.pos, L["kc"], L["vc"], pdl=True)
            if self.attention == "library":  # the framework's fused kernel, kept as a comparison for the benchmark
                valid = (torch.arange(self.T, device=self.dev) <= self.pos).view(1, 1, 1, self.T) if self.masked else None
                L["attn"].copy_(F.scaled_dot_product_attention(q.view(self.B, self.nq, 1, cfg.head_dim), L["kc"], L["vc"], attn_mask=valid,
                                                               enable_gqa=True).reshape(self.B, -1))
            else:
                ops.attn_decode(q, L["kc"], L["vc"], self.pos if self.masked else None, L["attn"], pdl=True)
            L["g_o"].run(pdl=True)
            self._allreduce(L["ob"])
            L["g_gu"].run(pdl=True)
            L["g_down"].run(pdl=True)
            self._allreduce(L["db"])
        ops.add_rmsnorm_(self.h, self.layers[-1]["db"], self.norm_f, self.xf, cfg.eps, pdl=True)
        self._greedy(self._head(self.xf, self.head_out, pdl=True))
        self.pos.add_(1)

    # ------------------------------------------------------------------ public
    def prefill(self, ids: torch.Tensor, all_logits: bool = False):
        """ids [B, S]: fills the KV cache for positions 0..S-1, leaves self.tok = greedy next token, pos = S.
        Returns the logits of the last position [B, vocab], or of every position [B, S, vocab] with `all_logits`."""
        cfg, B, d = self.cfg, self.B, self.cfg.head_dim
        S = ids.shape[1]
        if S > self.T:
            raise ValueError(f"prompt of {S} tokens exceeds the cache of {self.T}")
        x = self.embed[ids]  # [B, S, hidden]
        cos, sin = self.cos[:S], self.sin[:S]
        for L in self.layers:
            xn = _rms_norm(x, L["n1"], cfg.eps).reshape(B * S, cfg.hidden)
            q = ops.bitlinear(xn, *L["q"]).view(B, S, self.nq, d).transpose(1, 2)
            k = ops.bitlinear(xn, *L["k"]).view(B, S, self.nkv, d).transpose(1, 2)
            v = ops.bitlinear(xn, *L["v"]).view(B, S, self.nkv, d).transpose(1, 2)
            q, k = _rope(q, cos, sin), _rope(k, cos, sin)
            L["kc"][:, :, :S] = k
            L["vc"][:, :, :S] = v
            a = _causal_attention(q, k, v)
            a = a.transpose(1, 2).reshape(B * S, self.nq * d)
            if cfg.subln:
                a = _rms_norm(a, L["sa"], cfg.subln_eps)
            o = self._allreduce(ops.bitlinear(a, *L["o"]))
            x = x + o.view(B, S, cfg.hidden)
            hn = _rms_norm(x, L["n2"], cfg.eps).reshape(B * S, cfg.hidden)
            g, u = ops.bitlinear(hn, *L["gate"]), ops.bitlinear(hn, *L["up"])
            act = self._act(g, u)
            if cfg.subln:
                act = _rms_norm(act, L["sf"], cfg.subln_eps)
            dn = self._allreduce(ops.bitlinear(act, *L["down"]))
            x = x + dn.view(B, S, cfg.hidden)
        logits = self._head(_rms_norm(x if all_logits else x[:, -1], self.norm_f, cfg.eps))
        if self.tp > 1:  # the prompt pass returns the full rows
            parts = [torch.empty(*logits.shape[:-1], hi - lo, dtype=logits.dtype, device=logits.device)
                     for lo, hi in tpmod.shard_bounds(cfg.vocab, self.tp, 1)]
            dist.all_gather(parts, logits.contiguous(), group=self.group)
            logits = torch.cat(parts, -1)
        self.tok.copy_(logits[:, -1].argmax(-1) if all_logits else logits.argmax(-1))
        self.pos.fill_(S)
        self._pos_host = S
        return logits

    def capture(self, masked: bool = True, attention: str = "kernel"):
        """Warm up and capture the decode step as a CUDA graph.  `attention`: "kernel" (this library's decode
        attention) or "library" (the framework's fused attention, for comparison)."""
        self.masked = masked
        self.attention = attention
        pos0, tok0 = self.pos.clone(), self.tok.clone()
        s = torch.cuda.Stream()
        s.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(s):
            for _ in range(2):
                self._decode_step()
        torch.cuda.current_stream().wait_stream(s)
        torch.cuda.synchronize()
        self.graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.graph):
            self._decode_step()
        self.pos.copy_(pos0)
        self.tok.copy_(tok0)

    def release(self):
        """Drop the captured step graph.  A graph of a tensor-parallel step holds the communicator of its collectives:
        a process group is destroyed only after every such graph has been released."""
        if self.graph is not None:
            torch.cuda.synchronize()
            self.graph = None

    def decode(self, steps: int):
        """Greedy decoding of `steps` tokens per sequence; returns [B, steps] token ids."""
        if self._pos_host + steps > self.T:  # the cache and the rotary table hold T positions
            raise ValueError(f"decoding {steps} tokens from position {self._pos_host} exceeds the context of {self.T}")
        self._pos_host += steps
        out = []
        for _ in range(steps):
            self.graph.replay()
            self.tok.copy_(self.next_tok)
            out.append(self.next_tok.clone())
        return torch.stack(out, 1)

    def weight_bytes_per_step(self) -> int:
        """Bytes this rank streams per decode step: packed projections + bf16 lm_head + the KV cache."""
        cfg, d = self.cfg, self.cfg.head_dim
        packed = sum(L[n][0].numel() for L in self.layers for n in ("q", "k", "v", "o", "gate", "up", "down"))
        kv = 2 * len(self.layers) * self.B * self.nkv * self.T * d * 2
        return packed + self.lm_head.numel() * 2 + kv
