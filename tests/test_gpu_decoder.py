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
