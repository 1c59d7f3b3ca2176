"""Tensor-parallel BitLinear on two GPUs over NCCL (skipped with fewer than two devices).  Each rank is a child
process; the CUDA kernels run on its own GPU.  Column-parallel shards reproduce the single-GPU result exactly;
row-parallel partial sums are checked per shard bit for bit against the oracle, the reduced output within the
normalised tolerance."""
import datetime
import os
import sys
import time
import traceback

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
pytestmark = pytest.mark.gpu


def _worker(rank, world, port, results):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev, timeout=datetime.timedelta(seconds=120))
    try:
        from __graft_entry__ import load_package
        from oracle import bitlinear_oracle as O

        wf = load_package()
        from wrinklefree_monorepo_b200 import tp

        def at(stage):  # where a rank that never finishes had got to
            results[f"at{rank}"] = stage

        g = torch.Generator().manual_seed(0)
        n, k, m = 512, 1344, 6  # K = 21 units of 64: uneven split
        w = torch.randn(n, k, generator=g) * 0.02
        x = torch.randn(m, k, generator=g).bfloat16()
        codes, scale = wf.pack_ternary(w.to(dev))
        full = wf.bitlinear(x.to(dev), codes, scale, out_dtype=torch.float32)

        at("column/row parallel")
        col = tp.ColumnParallelBitLinear(codes, scale, k, n, gather_output=True)
        y = col(x.to(dev), out_dtype=torch.float32)
        assert torch.equal(y, full)

        row = tp.RowParallelBitLinear(codes, scale, k, n, input_is_parallel=False, reduce_dtype=torch.float32)
        lo, hi = row.bounds[rank]
        # this shard's integer accumulators against the oracle on the same slice
        _, acc = wf.bitlinear(x.to(dev)[:, lo:hi].contiguous(), row.codes, scale, want_acc=True)
        t = O.unpack_wf16(codes.cpu().numpy())[:, lo:hi]
        q, _ = O.act_quant_per_token(x.float().numpy()[:, lo:hi], "bf16")
        assert np.array_equal(acc.cpu().numpy(), O.int_gemm(q, t))
        y = row(x.to(dev), out_dtype=torch.float32)
        err = float((y - full).abs().max() / full.abs().max())
        assert err < 2e-2, err
        # the peer-memory all-reduce: equal to the fp32 sum in rank order on every rank, in place, repeatedly (the two
        # exchange slots alternate), also inside a CUDA graph; a row-parallel layer built on it
        at("one-shot all-reduce")
        ar = tp.OneShotAllReduce(max_bytes=1 << 20)
        for rep, (numel, dt) in enumerate([(4096, torch.bfloat16), (8, torch.bfloat16), (262144, torch.bfloat16), (4096, torch.float32),
                                           (520, torch.float16), (4096, torch.bfloat16)]):
            parts = [(torch.randn(numel, generator=torch.Generator().manual_seed(100 * rep + r)) * 3).to(dt) for r in range(world)]
            want = sum(p_.float() for p_ in parts).to(dt)
            y = parts[rank].to(dev)
            ar(y)
            assert torch.equal(y.cpu(), want), (rep, numel, dt)
        y = torch.ones(4096, dtype=torch.bfloat16, device=dev)
        graph = torch.cuda.CUDAGraph()
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            ar(y)
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        with torch.cuda.graph(graph):
            ar(y, pdl=True)
        for _ in range(3):
            graph.replay()
        torch.cuda.synchronize()
        assert torch.equal(y.cpu(), torch.full((4096,), float(world ** 4), dtype=torch.bfloat16))
        ar.status()
        row2 = tp.RowParallelBitLinear(codes, scale, k, n, input_is_parallel=False, reduce_dtype=torch.float32, all_reduce=ar)
        y2 = row2(x.to(dev), out_dtype=torch.float32)
        assert float((y2 - full).abs().max() / full.abs().max()) < 2e-2
        gathered = [torch.empty_like(y2) for _ in range(world)]
        dist.all_gather(gathered, y2)
        assert all(torch.equal(gathered[0], t_) for t_ in gathered)  # identical bits on every rank
        ar.status()
        # ---- a peer that does not take part: the wait runs out after a fraction of a second, the kernel returns, the host
        # reads the status, the group re-synchronises and the next all-reduce is right again (no fault is provoked: the
        # waiting kernel polls a flag that nobody sets and gives up)
        at("bounded wait")
        dist.barrier()
        y = torch.ones(4096, dtype=torch.bfloat16, device=dev)
        if rank == 0:
            ar(y)  # rank 1 sits this one out
        torch.cuda.synchronize()
        timed_out = False
        try:
            ar.status()
        except RuntimeError as e:
            timed_out = "ran out" in str(e)
        assert timed_out == (rank == 0), (rank, timed_out)
        ar.resync()
        for rep in range(3):
            y = torch.full((4096,), float(rank + 1 + rep), dtype=torch.bfloat16, device=dev)
            ar(y)
            assert torch.equal(y.cpu(), torch.full((4096,), float(sum(r + 1 + rep for r in range(world))), dtype=torch.bfloat16)), rep
        ar.status()
        wf.device_status()
        # ---- the exchange fused into the row-parallel projection: the launch pushes its partial output to every rank, the
        # residual add + RMSNorm sums what was pushed.  Same bits as projection -> peer-memory all-reduce -> add + RMSNorm;
        # both kernel forms (a single layer: 16 warps share an item; 152 problems in the launch: streaming),
        # several rounds (the two slots alternate).
        at("fused exchange")
        xp = ar.xchg_ptr()
        assert xp is not None
        for (n2, k2, m2, extra) in [(512, 1344, 1, 0), (512, 1344, 5, 0), (512, 1344, 2, 151)]:
            g2 = torch.Generator().manual_seed(n2 + m2)
            w2 = torch.randn(n2, k2, generator=g2) * 0.02
            c2, s2 = wf.pack_ternary(w2.to(dev))
            lo2, hi2 = tp.shard_bounds(k2, world, 64)[rank]
            shard = tp.shard_codes_k(c2, lo2, hi2)
            wn = (torch.rand(n2, generator=g2) + 0.5).bfloat16().to(dev)
            for rep in range(3):
                xs = torch.randn(m2, k2, generator=g2).bfloat16()[:, lo2:hi2].contiguous().to(dev)
                h0 = torch.randn(m2, n2, generator=g2).bfloat16().to(dev)
                # unfused: projection, peer-memory all-reduce, residual add + RMSNorm
                part = wf.bitlinear(xs, shard, s2, out_dtype=torch.bfloat16)
                ar(part)
                h_ref, y_ref = h0.clone(), torch.empty_like(h0)
                wf.ops.add_rmsnorm_(h_ref, part, wn, y_ref, 1e-5)
                # fused
                out = torch.empty(m2, n2, dtype=torch.bfloat16, device=dev)
                # `extra` more problems in the launch (plain ones: thousands of items put it on the streaming form)
                scratch = [torch.empty(m2, n2, dtype=torch.bfloat16, device=dev) for _ in range(extra)]
                grp = wf.DecodeGroup([dict(x=xs, codes=shard, w_scale=s2, out=out, xchg=xp)] +
                                     [dict(x=xs, codes=shard, w_scale=s2, out=o_) for o_ in scratch])
                grp.run(pdl=True)
                h_f, y_f = h0.clone(), torch.empty_like(h0)
                ar.reduce_add_rmsnorm_(h_f, wn, y_f, 1e-5, pdl=True)
                torch.cuda.synchronize()
                assert torch.equal(h_f, h_ref) and torch.equal(y_f, y_ref), (n2, m2, extra, rep)
                assert all(torch.equal(o_, out) for o_ in scratch)
        ar.status()
        wf.device_status()
        # ---- the decoder: heads, MLP width and the output head sharded over the ranks, against one rank on its own
        from wrinklefree_monorepo_b200.decoder import DecoderConfig, TernaryDecoder

        at("decoder build")
        solo = [dist.new_group([r]) for r in range(world)][rank]  # collective: every rank creates every group
        cfg = DecoderConfig(layers=2, hidden=256, n_q=4, n_kv=2, head_dim=64, intermediate=512, vocab=1000)
        ids = torch.randint(0, cfg.vocab, (3, 9), generator=torch.Generator().manual_seed(5)).to(dev)
        m_tp = TernaryDecoder(cfg, 3, 16, dev, seed=3)
        m_1 = TernaryDecoder(cfg, 3, 16, dev, seed=3, group=solo)
        assert m_tp.tp == world and m_1.tp == 1 and m_tp.lm_head.shape[0] == cfg.vocab // world
        at("decoder prefill")
        l_tp, l_1 = m_tp.prefill(ids).float(), m_1.prefill(ids).float()
        assert l_tp.shape == l_1.shape
        assert float((l_tp - l_1).abs().max() / l_1.abs().max()) < 3e-2  # row-parallel layers quantize their K slices locally
        at("decoder capture")
        m_tp.capture(masked=True)
        m_1.capture(masked=True)
        at("decoder decode")
        toks_tp, toks_1 = m_tp.decode(4), m_1.decode(4)
        at("decoder checks")
        both = [torch.empty_like(toks_tp) for _ in range(world)]
        dist.all_gather(both, toks_tp)
        assert all(torch.equal(both[0], t_) for t_ in both)  # every rank picked the same tokens
        assert int(toks_tp.max()) < cfg.vocab and (toks_tp == toks_1).float().mean() >= 0.5
        # the sharded head's greedy pick equals the arg-max of the gathered rows
        full = [torch.empty_like(m_tp.logits) for _ in range(world)]
        dist.all_gather(full, m_tp.logits.contiguous())
        assert torch.equal(torch.cat(full, -1).float().argmax(-1), m_tp.next_tok)
        # the fused exchange (the default from two sequences on) against the exchange as a kernel of its own: same bits
        assert m_tp.fuse_exchange
        m_sep = TernaryDecoder(cfg, 3, 16, dev, seed=3, fuse_exchange=False)
        assert not m_sep.fuse_exchange
        m_sep.prefill(ids)
        m_sep.capture(masked=True)
        toks_sep = m_sep.decode(4)
        assert torch.equal(toks_sep, toks_tp) and torch.equal(m_sep.logits, m_tp.logits)
        wf.device_status()
        results[rank] = "ok"
    except BaseException:
        # the peer may be inside a collective: report and leave without the orderly teardown; the parent ends the other rank
        results[rank] = traceback.format_exc()
        os._exit(1)
    # captured steps hold the communicator of their collectives: release them before the group goes away
    at("teardown")
    m_tp.release()
    m_1.release()
    m_sep.release()
    dist.destroy_process_group()
    at("done")


def test_tp2_nccl():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    mgr = mp.Manager()
    results = mgr.dict()
    ctx = mp.spawn(_worker, args=(2, 29650 + os.getpid() % 300, results), nprocs=2, join=False)
    deadline = time.time() + 300
    try:
        while not ctx.join(timeout=5):
            if time.time() > deadline:
                for p in ctx.processes:  # exactly the two children started above
                    if p.is_alive():
                        p.kill()
                pytest.fail(f"ranks still running after 300 s; reported so far: {dict(results)}")
    except Exception as e:  # a rank left with an error: show what it recorded
        pytest.fail(f"{e}\n{dict(results)}")
    assert {r: results.get(r) for r in (0, 1)} == {0: "ok", 1: "ok"}, dict(results)
