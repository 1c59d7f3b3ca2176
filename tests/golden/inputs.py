"""Seeded synthetic inputs shared by the golden-vector generator and the tests.

Everything is drawn from torch's CPU generator with an explicit seed, so the
generator script (run where the reference is installed) and the tests (run
anywhere) see the same tensors; each golden file stores a SHA-256 of its inputs
and the tests compare it before trusting the stored outputs.
"""
from __future__ import annotations

import hashlib

import numpy as np
import torch

# name -> (M tokens, K in_features, N out_features, seed)
CASES = {
    # BASELINE config 1: SmolLM2-135M MLP up-projection, seed 0
    "c1": (16, 576, 1536, 0),
    "k64": (3, 64, 32, 11),
    "k128": (1, 128, 48, 12),
    "k192": (5, 192, 80, 13),
    "k512": (8, 512, 128, 14),
    "k1024": (2, 1024, 64, 15),
}
# shapes whose K is a multiple of 128 also go through the reference's I2_S CPU kernel
I2S_CASES = ["k128", "k512", "k1024"]


def make_inputs(name: str):
    """Returns (x fp32 [M,K] ~ N(0,1), w fp32 [N,K] ~ N(0,0.02)) as torch CPU tensors."""
    m, k, n, seed = CASES[name]
    g = torch.Generator().manual_seed(seed)
    w = torch.randn(n, k, generator=g, dtype=torch.float32) * 0.02
    x = torch.randn(m, k, generator=g, dtype=torch.float32)
    return x, w


def with_outliers(x: torch.Tensor, seed: int, frac: float = 1e-3, mag: float = 20.0) -> torch.Tensor:
    """Activation distribution of the decode/prefill sweeps: N(0,1) with a `frac`
    share of entries replaced by +-mag."""
    g = torch.Generator().manual_seed(seed + 7919)
    mask = torch.rand(x.shape, generator=g) < frac
    sign = torch.where(torch.rand(x.shape, generator=g) < 0.5, -1.0, 1.0)
    return torch.where(mask, sign * mag, x)


def sha(*arrays) -> str:
    h = hashlib.sha256()
    for a in arrays:
        h.update(np.ascontiguousarray(a).tobytes())
    return h.hexdigest()


# ---------------------------------------------------------------------------------------------
# A two-layer decoder at SmolLM2-135M widths (hidden 576, 9 query / 3 KV heads of 64, SwiGLU-shaped MLP of 1536)
# with a small vocabulary, for the whole-model parity fixtures.
MODEL_CFG = dict(layers=2, hidden=576, n_q=9, n_kv=3, head_dim=64, intermediate=1536, vocab=1024, rope_theta=1e5,
                 norm_eps=1e-6, max_pos=64)
MODEL_BATCH, MODEL_PROMPT, MODEL_STEPS = 2, 24, 3  # ids [B, PROMPT + STEPS]; the last STEPS tokens are teacher-forced decode steps
MODEL_KEEP_FROM = 0                                # logits are stored for positions KEEP_FROM .. PROMPT + STEPS - 1


def model_weights(seed: int = 31):
    """Seeded fp32 weights of the fixture decoder: dict name -> tensor, names after the reference's modules.
    Projections ~ N(0, 0.02); norm weights ~ 1 + 0.1 N(0, 1) so that every norm matters to the result."""
    c = MODEL_CFG
    g = torch.Generator().manual_seed(seed)

    def lin(n, k):
        return torch.randn(n, k, generator=g, dtype=torch.float32) * 0.02

    def norm(n):
        return 1.0 + 0.1 * torch.randn(n, generator=g, dtype=torch.float32)

    d, h, it = c["head_dim"], c["hidden"], c["intermediate"]
    w = {"embed_tokens.weight": lin(c["vocab"], h), "lm_head.weight": lin(c["vocab"], h), "transformer.norm.weight": norm(h)}
    for i in range(c["layers"]):
        p = f"transformer.layers.{i}."
        w[p + "input_layernorm.weight"] = norm(h)
        w[p + "self_attn.q_proj.weight"] = lin(c["n_q"] * d, h)
        w[p + "self_attn.k_proj.weight"] = lin(c["n_kv"] * d, h)
        w[p + "self_attn.v_proj.weight"] = lin(c["n_kv"] * d, h)
        w[p + "self_attn.subln.weight"] = norm(c["n_q"] * d)
        w[p + "self_attn.o_proj.weight"] = lin(h, c["n_q"] * d)
        w[p + "post_attention_layernorm.weight"] = norm(h)
        w[p + "mlp.gate_proj.weight"] = lin(it, h)
        w[p + "mlp.up_proj.weight"] = lin(it, h)
        w[p + "mlp.subln.weight"] = norm(it)
        w[p + "mlp.down_proj.weight"] = lin(h, it)
    return w


def model_ids(seed: int = 32) -> torch.Tensor:
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, MODEL_CFG["vocab"], (MODEL_BATCH, MODEL_PROMPT + MODEL_STEPS), generator=g)
