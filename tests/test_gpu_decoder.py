"""Decoder harness: the CUDA-graphed decode step (KV cache, RoPE, masking, grouped projections) must agree
with the prefill pass over the same tokens, which takes the other kernel path for every projection."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_stepwise_decode_matches_prefill(wf):
    from wrinklefree_monorepo_b200.decoder import DecoderConfig, TernaryDecoder

    cfg = DecoderConfig(layers=2, hidden=256, n_q=4, n_kv=2, head_dim=64, intermediate=512, vocab=1000)
    dev = torch.device("cuda", 0)
    B, S, T = 3, 9, 16
    g = torch.Generator().manual_seed(5)
    ids = torch.randint(0, cfg.vocab, (B, S), generator=g).to(dev)

    m1 = TernaryDecoder(cfg, B, T, dev, seed=1)
    ref = m1.prefill(ids).float()
    assert int(m1.pos) == S

    m2 = TernaryDecoder(cfg, B, T, dev, seed=1)
    m2.capture(masked=True)
    assert int(m2.pos) == 0
    for t in range(S):
        m2.tok.copy_(ids[:, t])
        m2.graph.replay()
    torch.cuda.synchronize()
    got = m2.logits.float()
    assert int(m2.pos) == S
    err = float((got - ref).abs().max() / ref.abs().max())
    assert err < 3e-2, err
    assert (got.argmax(-1) == ref.argmax(-1)).float().mean() >= 2 / 3
    # the caches hold the same keys
    kerr = float((m1.layers[0]["kc"][:, :, :S].float() - m2.layers[0]["kc"][:, :, :S].float()).abs().max())
    assert kerr < 2e-2, kerr
    # greedy continuation runs and stays in range
    out = m2.decode(4)
    assert out.shape == (B, 4) and int(out.max()) < cfg.vocab
    wf.device_status()


def test_fused_elementwise_kernels(wf):
    from wrinklefree_monorepo_b200 import ops

    dev = torch.device("cuda", 0)
    g = torch.Generator().manual_seed(3)
    M, K = 5, 576
    h = torch.randn(M, K, generator=g).bfloat16().to(dev)
    delta = torch.randn(M, K, generator=g).bfloat16().to(dev)
    w = (1 + 0.1 * torch.randn(K, generator=g)).bfloat16().to(dev)
    want_h = (h + delta)
    v = want_h.float()
    want_y = (v * torch.rsqrt(v.pow(2).mean(-1, keepdim=True) + 1e-5)).to(torch.bfloat16) * w
    y = torch.empty_like(h)
    h2 = h.clone()
    ops.add_rmsnorm_(h2, delta, w, y, 1e-5)
    assert torch.equal(h2, want_h)
    assert float((y.float() - want_y.float()).abs().max()) <= 2e-2 * float(want_y.float().abs().max())
    y0 = torch.empty_like(h)
    ops.add_rmsnorm_(h2, None, w, y0, 1e-5)
    assert torch.equal(y0, y)

    gate = torch.randn(4, 512, generator=g).bfloat16().to(dev)
    up = torch.randn(4, 512, generator=g).bfloat16().to(dev)
    out = torch.empty_like(gate)
    ops.act_mul(gate, up, out, "silu")
    ref = torch.nn.functional.silu(gate) * up
    assert float((out.float() - ref.float()).abs().max()) <= 2e-2 * float(ref.float().abs().max())
    ops.act_mul(gate, up, out, "relu2")
    ref = torch.relu(gate).pow(2) * up
    assert float((out.float() - ref.float()).abs().max()) <= 2e-2 * float(ref.float().abs().max())

    B, nq, nkv, D, T = 3, 4, 2, 64, 16
    q = torch.randn(B, nq * D, generator=g).bfloat16().to(dev)
    k = torch.randn(B, nkv * D, generator=g).bfloat16().to(dev)
    vv = torch.randn(B, nkv * D, generator=g).bfloat16().to(dev)
    inv = 1.0 / (1e4 ** (torch.arange(0, D, 2, dtype=torch.float32) / D))
    ang = torch.arange(T, dtype=torch.float32)[:, None] * inv[None, :]
    cos, sin = ang.cos().to(dev), ang.sin().to(dev)
    pos = torch.tensor(21, dtype=torch.long, device=dev)  # slot 21 % 16 = 5
    kc = torch.zeros(B, nkv, T, D, dtype=torch.bfloat16, device=dev)
    vc = torch.zeros_like(kc)

    def rope(x, c, s):
        x1, x2 = x[..., : D // 2].float(), x[..., D // 2 :].float()
        return torch.cat([x1 * c - x2 * s, x2 * c + x1 * s], -1).to(torch.bfloat16)

    want_q = rope(q.view(B, nq, D), cos[5], sin[5]).reshape(B, nq * D)
    want_k = rope(k.view(B, nkv, D), cos[5], sin[5])
    ops.rope_kv_(q, k, vv, cos, sin, pos, kc, vc)
    assert torch.equal(q, want_q)
    assert torch.equal(kc[:, :, 5], want_k) and torch.equal(vc[:, :, 5], vv.view(B, nkv, D))
    assert not kc[:, :, 4].any() and not kc[:, :, 6].any()
