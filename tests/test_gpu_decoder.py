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


# ---------------------------------------------------------------- against the reference's own model
import os  # noqa: E402

import numpy as np  # noqa: E402

import inputs as gi  # noqa: E402

GOLD = os.path.join(os.path.dirname(__file__), "golden")


def _fixture_decoder(act, dtype, pack_mode):
    from wrinklefree_monorepo_b200.decoder import DecoderConfig, TernaryDecoder

    c = gi.MODEL_CFG
    z = np.load(os.path.join(GOLD, f"model_{act}.npz"))
    weights, ids = gi.model_weights(), gi.model_ids()
    assert gi.sha(ids.numpy(), *[weights[k].numpy() for k in sorted(weights)]) == str(z["input_sha"])
    cfg = DecoderConfig(layers=c["layers"], hidden=c["hidden"], n_q=c["n_q"], n_kv=c["n_kv"], head_dim=c["head_dim"],
                        intermediate=c["intermediate"], vocab=c["vocab"], rope_theta=c["rope_theta"], act=act,
                        eps=c["norm_eps"], subln=True)
    dev = torch.device("cuda", 0)
    model = TernaryDecoder(cfg, gi.MODEL_BATCH, c["max_pos"], dev, dtype=dtype, weights=weights, pack_mode=pack_mode)
    return model, ids.to(dev), z


def _nerr(got, ref):
    return float(np.abs(got - ref).max() / np.abs(ref).max())


@pytest.mark.parametrize("act", ["relu2", "silu"])
def test_prefill_equals_reference_model_fp32(wf, act):
    """TernaryDecoder.prefill on the weights of the reference's BitNetLlama (2 layers at SmolLM2-135M widths, SubLN,
    GQA, interleaved RoPE) against the reference's own fp32 forward, per position, err = max|a-b| / max|b|.

    Rounding to int8 is discontinuous: an input that lands within a few 1e-7 of a rounding boundary is rounded the
    other way when the fp32 summation order of a norm differs, that one code moves the token's hidden state by
    ~1e-3, and the next quantizations amplify it to ~1e-2 at the logits.  The reference does this to itself: adding
    3e-7 relative noise to its embeddings left 44 of 54 positions within 5e-7 and moved the other 10 by 0.5-1.7 %.
    So: at least 60 % of the positions must agree to 1e-5 (the computation is the same one), and no position may be
    off by more than 3e-2 (a rounding cascade, not a different model)."""
    model, ids, z = _fixture_decoder(act, torch.float32, torch.float32)
    logits = model.prefill(ids, all_logits=True)
    got = logits[:, gi.MODEL_KEEP_FROM:].float().cpu().numpy()
    ref = z["logits_f32"]
    err = np.abs(got - ref).max(-1) / np.abs(ref).max()  # [batch, position]
    np.set_printoptions(precision=1, linewidth=250)
    print(f"fp32 {act}: per-position error\n{err}")
    # A position's result depends on every earlier position of its sequence through attention, so a cascade, once
    # started, reaches the later positions of that sequence.  Measured: 45 / 36 of the 54 positions (relu2 / silu)
    # agree to 1e-6, the others sit at 5e-4 .. 1.7e-2.
    assert (err <= 1e-5).mean() >= 0.6, (err <= 1e-5).mean()
    assert err.max() <= 3e-2, err.max()
    assert (got.argmax(-1) == ref.argmax(-1)).mean() >= 0.9
    wf.device_status()


@pytest.mark.parametrize("act", ["relu2", "silu"])
def test_bf16_prefill_and_decode_steps_follow_reference_model(wf, act):
    """bf16 end to end, weights ternarized by the cast-first rule of BitLinear.forward.  Held to the reference's bf16
    forward within max|a-b| / max|b| <= 6e-2 (measured 0.037-0.041): the reference evaluates its norms, residuals and
    attention in bf16 arithmetic, this decoder in fp32 with one rounding, so int8 codes near a rounding boundary differ
    and the random two-layer network amplifies that.  For scale: the reference's own bf16 and fp32 forwards differ by
    0.16 on this fixture, and this decoder must sit as close to the bf16 reference as that (checked as well).  The
    CUDA-graphed decode step (fused norm, RoPE + cache write, grouped projections) is then teacher-forced over the next
    positions and held to the same logits."""
    model, ids, z = _fixture_decoder(act, torch.bfloat16, torch.bfloat16)
    S, K0 = gi.MODEL_PROMPT, gi.MODEL_KEEP_FROM
    logits = model.prefill(ids[:, :S], all_logits=True)
    got = logits[:, K0:].float().cpu().numpy()
    e_bf16, e_f32 = _nerr(got, z["logits_bf16"][:, :S - K0]), _nerr(got, z["logits_f32"][:, :S - K0])
    print(f"prefill {act}: vs bf16 reference {e_bf16:.4f}, vs fp32 reference {e_f32:.4f}")
    ref_gap = _nerr(z["logits_bf16"], z["logits_f32"])  # what bf16 arithmetic alone costs the reference
    assert e_bf16 <= 6e-2 and e_bf16 < ref_gap / 2 and e_f32 <= 1.5 * ref_gap, (e_bf16, e_f32, ref_gap)
    model.capture(masked=True)
    for i in range(gi.MODEL_STEPS):
        model.tok.copy_(ids[:, S + i])
        model.graph.replay()
        torch.cuda.synchronize()
        step = model.logits.float().cpu().numpy()
        e1, e2 = _nerr(step, z["logits_bf16"][:, S - K0 + i]), _nerr(step, z["logits_f32"][:, S - K0 + i])
        print(f"step {i} {act}: vs bf16 reference {e1:.4f}, vs fp32 reference {e2:.4f}")
        assert e1 <= 6e-2 and e2 <= 1.5 * ref_gap, (i, e1, e2)
    wf.device_status()


@pytest.mark.parametrize("B,nq,nkv,D,T,pos", [(1, 32, 8, 128, 2080, 2047), (3, 9, 3, 64, 100, 37), (32, 32, 8, 128, 300, 299),
                                              (2, 4, 4, 64, 64, 0), (5, 8, 1, 128, 1000, None), (7, 6, 2, 64, 130, 128), (300, 8, 4, 128, 70, 69)])
def test_decode_attention_kernel(wf, B, nq, nkv, D, T, pos):
    """The decode-step attention kernel (grouped-query heads, context split over CTAs and merged in the launch, bf16
    cache) against fp32 softmax attention over the valid positions: max|a-b| / max|b| <= 1e-2 (the probabilities are
    rounded to bf16 in front of the second product, the output is bf16).  Positions beyond the valid length hold
    large garbage that must not leak in."""
    from wrinklefree_monorepo_b200 import ops

    dev = torch.device("cuda", 0)
    g = torch.Generator().manual_seed(B * 1000 + T)
    q = torch.randn(B, nq * D, generator=g).bfloat16().to(dev)
    kc = torch.randn(B, nkv, T, D, generator=g).bfloat16().to(dev)
    vc = torch.randn(B, nkv, T, D, generator=g).bfloat16().to(dev)
    n_valid = T if pos is None else pos + 1
    kc[:, :, n_valid:] = 1e4
    vc[:, :, n_valid:] = -1e4
    out = torch.empty(B, nq * D, dtype=torch.bfloat16, device=dev)
    pos_t = None if pos is None else torch.tensor(pos, dtype=torch.long, device=dev)
    for _ in range(2):  # the merge tickets must be reusable
        out.fill_(7)
        ops.attn_decode(q, kc, vc, pos_t, out)
        qf = q.float().view(B, nkv, nq // nkv, D)
        kf, vf = kc.float()[:, :, :n_valid], vc.float()[:, :, :n_valid]
        s = torch.einsum("bhgd,bhtd->bhgt", qf, kf) * D ** -0.5
        ref = torch.einsum("bhgt,bhtd->bhgd", torch.softmax(s, -1), vf).reshape(B, nq * D)
        err = float((out.float() - ref).abs().max() / ref.abs().max())
        assert err <= 1e-2, err


def test_fused_inputs_of_grouped_projections(wf, oracle_c):
    """The fused input modes of the grouped decode kernel against the unfused kernels of the library: rmsnorm(x + x2)
    in front of a q/k/v-like group (all three forms of the kernel: shared tokens, a single matrix, a streaming
    stack), and act(gate) * up in front of a down-like projection.  Activation modes: accumulators and outputs
    identical to the unfused chain.  Norm mode: the residual output identical; the projection outputs within 1e-2
    (the mean of squares is summed in another order, which may move single int8 codes)."""
    from wrinklefree_monorepo_b200 import ops

    dev = torch.device("cuda", 0)
    g = torch.Generator().manual_seed(11)
    for (m, k, ns) in ((1, 4096, (4096, 1024, 1024)), (5, 576, (576, 192, 192)), (3, 2560, (6912,)), (20, 640, (512, 512))):
        h = torch.randn(m, k, generator=g).bfloat16().to(dev)
        delta = torch.randn(m, k, generator=g).bfloat16().to(dev)
        w = (1 + 0.1 * torch.randn(k, generator=g)).bfloat16().to(dev)
        mats = [wf.pack_ternary((torch.randn(n, k, generator=g) * 0.02).to(dev)) for n in ns]
        for with_delta in (True, False):
            # unfused: norm kernel, then the group on its output
            h_ref = h.clone()
            xn = torch.empty_like(h)
            ops.add_rmsnorm_(h_ref, delta if with_delta else None, w, xn, 1e-5)
            ref = ops.DecodeGroup([dict(x=xn, codes=c, w_scale=s_, out_dtype=torch.float32) for c, s_ in mats]).run()
            h_out = torch.zeros_like(h)
            probs = [dict(x=h, x2=delta if with_delta else None, x_mode="norm", norm_w=w, norm_eps=1e-5, codes=c, w_scale=s_,
                          out_dtype=torch.float32, h_out=h_out if i == 0 else None) for i, (c, s_) in enumerate(mats)]
            grp = ops.DecodeGroup(probs)
            for pdl in (False, True):
                h_out.zero_()
                got = grp.run(pdl=pdl)
                assert torch.equal(h_out, h_ref), (m, k, with_delta)
                for a, b in zip(got, ref):
                    err = float((a - b).abs().max() / b.abs().max())
                    assert err <= 1e-2, (m, k, with_delta, err)
    # a streaming stack (thousands of row items) with the norm fused in
    m, k = 2, 1024
    h = torch.randn(m, k, generator=g).bfloat16().to(dev)
    w = (1 + 0.1 * torch.randn(k, generator=g)).bfloat16().to(dev)
    mats = [wf.pack_ternary((torch.randn(6000 + 16 * i, k, generator=g) * 0.02).to(dev)) for i in range(8)]
    xn = torch.empty_like(h)
    ops.add_rmsnorm_(h.clone(), None, w, xn, 1e-6)
    ref = ops.DecodeGroup([dict(x=xn, codes=c, w_scale=s_, out_dtype=torch.float32) for c, s_ in mats]).run()
    got = ops.DecodeGroup([dict(x=h, x_mode="norm", norm_w=w, norm_eps=1e-6, codes=c, w_scale=s_, out_dtype=torch.float32) for c, s_ in mats]).run(pdl=True)
    for a, b in zip(got, ref):
        assert float((a - b).abs().max() / b.abs().max()) <= 1e-2
    # activation modes: bit-exact against act_mul + projection
    for (m, k, n, mode) in ((1, 14336, 4096, "silu"), (4, 1536, 576, "relu2"), (9, 1024, 300, "silu"), (33, 640, 128, "relu2")):
        gate = torch.randn(m, k, generator=g).bfloat16().to(dev)
        up = torch.randn(m, k, generator=g).bfloat16().to(dev)
        codes, sc = wf.pack_ternary((torch.randn(n, k, generator=g) * 0.02).to(dev))
        act = torch.empty_like(gate)
        ops.act_mul(gate, up, act, mode)
        y_ref, acc_ref = wf.bitlinear(act, codes, sc, out_dtype=torch.float32, want_acc=True, path="decode")
        grp = ops.DecodeGroup([dict(x=gate, x2=up, x_mode=mode, codes=codes, w_scale=sc, out_dtype=torch.float32, want_acc=True)])
        y = grp.run()[0]
        assert torch.equal(grp.accs[0], acc_ref) and torch.equal(y, y_ref), (m, k, n, mode)
    wf.device_status()


def test_fused_decode_step_equals_unfused(wf):
    """The six-launch decode step (fused inputs) against the ten-launch step of the same model."""
    from wrinklefree_monorepo_b200.decoder import DecoderConfig, TernaryDecoder

    cfg = DecoderConfig(layers=3, hidden=256, n_q=4, n_kv=2, head_dim=64, intermediate=512, vocab=1000)
    dev = torch.device("cuda", 0)
    B, S, T = 3, 7, 16
    ids = torch.randint(0, cfg.vocab, (B, S), generator=torch.Generator().manual_seed(6)).to(dev)
    outs = []
    for fuse in (True, False):
        m = TernaryDecoder(cfg, B, T, dev, seed=2, fuse=fuse)
        assert m.fused == fuse
        m.capture(masked=True)
        steps = []
        for t in range(S):
            m.tok.copy_(ids[:, t])
            m.graph.replay()
            steps.append(m.logits.float().clone())
        outs.append(torch.stack(steps))
    err = float((outs[0] - outs[1]).abs().max() / outs[1].abs().max())
    assert err <= 2e-2, err
    assert (outs[0].argmax(-1) == outs[1].argmax(-1)).float().mean() >= 0.9
    wf.device_status()


@pytest.mark.parametrize("m,n,k", [(1, 1000, 576), (3, 130, 72), (32, 5000, 4096), (256, 3000, 4096), (300, 1100, 1024), (17, 128, 8)])
@pytest.mark.parametrize("out_dtype", [torch.bfloat16, torch.float32])
def test_linear_bf16_output_head(wf, m, n, k, out_dtype):
    """The bf16 linear kernel (the decoder's output head) against an fp32 matmul of the same bf16 operands: the products
    are exact in fp32, only the order of the fp32 additions differs (tolerance 1e-3 of the largest output for f32, one
    bf16 rounding step more for bf16 outputs); row tails, token tails, K tails, more than 256 tokens."""
    dev = torch.device("cuda", 0)
    g = torch.Generator(device=dev).manual_seed(m * 1000 + n + k)
    x = torch.randn(m, k, generator=g, device=dev).bfloat16()
    w = (torch.randn(n, k, generator=g, device=dev) * 0.05).bfloat16()
    ref = x.float() @ w.float().t()
    y = wf.linear_bf16(x, w, out_dtype=out_dtype)
    assert y.shape == (m, n) and y.dtype == out_dtype
    tol = 1e-3 if out_dtype == torch.float32 else 1e-2
    err = float((y.float() - ref).abs().max() / ref.abs().max())
    assert err < tol, err
    # strided views: rows of a wider buffer on both sides, and into a wider output
    if k >= 64:
        xw = torch.zeros(m, k + 16, dtype=torch.bfloat16, device=dev)
        xw[:, :k] = x
        ww = torch.zeros(n, k + 8, dtype=torch.bfloat16, device=dev)
        ww[:, :k] = w
        out = torch.full((m, n + 5), 7.0, dtype=out_dtype, device=dev)
        wf.linear_bf16(xw[:, :k], ww[:, :k], out=out[:, :n])
        assert torch.equal(out[:, :n], y) and bool((out[:, n:] == 7.0).all())
    wf.device_status()


def test_linear_bf16_rejects_what_it_cannot_run(wf):
    dev = torch.device("cuda", 0)
    x = torch.zeros(2, 64, dtype=torch.bfloat16, device=dev)
    w = torch.zeros(8, 64, dtype=torch.bfloat16, device=dev)
    with pytest.raises(ValueError):
        wf.linear_bf16(x.float(), w)
    with pytest.raises(RuntimeError):
        wf.linear_bf16(x[:, :60], w[:, :60])  # K not a multiple of 8


@pytest.mark.parametrize("m,k", [(1, 4096), (5, 576), (3, 14336), (2, 16384), (33, 2048)])
def test_norm_and_activation_with_fused_quantization(wf, m, k):
    """The residual add + RMSNorm and the gate activation that quantize their own result: int8 codes, per-token multipliers,
    the updated residual stream and the optional bf16 copy equal the unfused chain (kernel, then act_quant_i8) bit for bit."""
    from wrinklefree_monorepo_b200 import ops

    dev = torch.device("cuda", 0)
    g = torch.Generator(device=dev).manual_seed(m * 100 + k)
    h0 = torch.randn(m, k, generator=g, device=dev).bfloat16()
    delta = torch.randn(m, k, generator=g, device=dev).bfloat16()
    w = (torch.rand(k, generator=g, device=dev) + 0.5).bfloat16()
    for d in (delta, None):
        h_ref, y_ref = h0.clone(), torch.empty_like(h0)
        ops.add_rmsnorm_(h_ref, d, w, y_ref, 1e-5)
        q_ref, s_ref = wf.act_quant_i8(y_ref, eps=1e-5)
        h_f, y_f = h0.clone(), torch.empty_like(h0)
        q = torch.empty(m, k, dtype=torch.int8, device=dev)
        s = torch.empty(m, dtype=torch.float32, device=dev)
        ops.add_rmsnorm_quant_(h_f, d, w, q, s, 1e-5, out=y_f)
        assert torch.equal(h_f, h_ref) and torch.equal(y_f, y_ref) and torch.equal(q, q_ref) and torch.equal(s, s_ref)
        q2, s2 = torch.empty_like(q), torch.empty_like(s)
        ops.add_rmsnorm_quant_(h0.clone(), d, w, q2, s2, 1e-5)  # without the bf16 copy
        assert torch.equal(q2, q_ref) and torch.equal(s2, s_ref)
    up = torch.randn(m, k, generator=g, device=dev).bfloat16()
    for mode in ("silu", "relu2"):
        a_ref = ops.act_mul(h0, up, torch.empty_like(h0), mode)
        q_ref, s_ref = wf.act_quant_i8(a_ref, eps=1e-5)
        q = torch.empty(m, k, dtype=torch.int8, device=dev)
        s = torch.empty(m, dtype=torch.float32, device=dev)
        out = torch.empty_like(h0)
        ops.act_mul_quant(h0, up, q, s, mode, out=out)
        assert torch.equal(out, a_ref) and torch.equal(q, q_ref) and torch.equal(s, s_ref)
