"""Tensor-parallel sharding and reassembly on CPU ranks (gloo, world size 2).  The contraction itself is
stood in for by the CPU oracle here (the CUDA path is covered by the gpu-marked tests); what is checked is
the host logic: shard bounds, byte-slicing of packed weights, bias placement, the all-reduce and all-gather."""
import os
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def oracle_linear(x, codes, w_scale, bias=None, layout=0, out_dtype=None, **kw):
    """CPU stand-in with the signature of ops.bitlinear (test infrastructure only)."""
    from oracle import bitlinear_oracle as O

    unpack = O.unpack_i2s if layout == 1 else O.unpack_wf16
    t = unpack(codes.numpy())
    dt = {torch.float32: "f32", torch.bfloat16: "bf16", torch.float16: "f16"}[x.dtype]
    q, s = O.act_quant_per_token(x.float().numpy().reshape(-1, x.shape[-1]), dt)
    acc = O.int_gemm(q, t)
    ws = float(w_scale[0]) if isinstance(w_scale, torch.Tensor) else float(w_scale)
    y = O.rescale(acc, s, np.float32(ws), bias.float().numpy() if bias is not None else None)
    return torch.from_numpy(y).to(out_dtype or x.dtype).reshape(*x.shape[:-1], t.shape[0])


def _worker(rank, world, port, results):
    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from __graft_entry__ import load_package
        from oracle import bitlinear_oracle as O

        wf = load_package()
        from wrinklefree_monorepo_b200 import tp

        g = torch.Generator().manual_seed(0)
        n, k, m = 96, 448, 5  # K = 7 units of 64: uneven split over two ranks
        w = torch.randn(n, k, generator=g) * 0.02
        x = torch.randn(m, k, generator=g)
        bias = torch.randn(n, generator=g)
        t, s_w = O.ternarize_absmean(w.numpy())
        codes = torch.from_numpy(O.pack_wf16(t))
        full = oracle_linear(x, codes, float(s_w), bias=bias)

        col = tp.ColumnParallelBitLinear(codes, float(s_w), k, n, bias=bias, gather_output=True, linear_fn=oracle_linear)
        assert col.codes.shape == (n // world, k // 4)
        y = col(x)
        assert torch.equal(y, full)  # rows are independent: gathering the shards reproduces the full result exactly

        row = tp.RowParallelBitLinear(codes, float(s_w), k, n, bias=bias, input_is_parallel=False,
                                      linear_fn=oracle_linear)
        lo, hi = row.bounds[rank]
        assert (hi - lo) % 64 == 0 and row.codes.shape == (n, (hi - lo) // 4)
        assert np.array_equal(O.unpack_wf16(row.codes.numpy()), t[:, lo:hi])  # a byte slice is a K slice
        assert (row.bias is not None) == (rank == 0)
        y = row(x)
        # per-rank activation scales differ from the unsharded ones: equal within quantization noise
        err = float((y - full).abs().max() / full.abs().max())
        assert err < 2e-2, err
        # every rank holds the same reduced tensor
        ys = [torch.empty_like(y) for _ in range(world)]
        dist.all_gather(ys, y)
        assert torch.equal(ys[0], ys[1])
        # the peer-memory all-reduce needs GPUs: without them its wrapper falls back to the group's all_reduce, also
        # as the `all_reduce` hook of a row-parallel layer
        ar = tp.OneShotAllReduce()
        v = torch.full((8,), float(rank + 1))
        assert torch.equal(ar(v), torch.full((8,), 3.0))
        ar.status()
        row2 = tp.RowParallelBitLinear(codes, float(s_w), k, n, bias=bias, input_is_parallel=False, linear_fn=oracle_linear,
                                       all_reduce=ar)
        assert torch.equal(row2(x), y)
        results[rank] = "ok"
    finally:
        dist.destroy_process_group()


def test_tp_world_size_2_gloo():
    world = 2
    port = 29500 + os.getpid() % 1000
    mgr = mp.Manager()
    results = mgr.dict()
    mp.spawn(_worker, args=(world, port, results), nprocs=world, join=True)
    assert dict(results) == {0: "ok", 1: "ok"}


def test_shard_bounds():
    sys.path.insert(0, ROOT)
    from __graft_entry__ import load_package

    load_package()
    from wrinklefree_monorepo_b200 import tp

    b = tp.shard_bounds(6912, 8, 64)  # 108 units over 8 ranks: 14,14,14,14,13,13,13,13
    assert b[0] == (0, 896) and b[-1][1] == 6912 and all((hi - lo) % 64 == 0 for lo, hi in b)
    assert sorted({hi - lo for lo, hi in b}) == [832, 896]
    assert tp.shard_bounds(4096, 8, 16) == [(i * 512, (i + 1) * 512) for i in range(8)]
    with pytest.raises(ValueError):
        tp.shard_bounds(100, 2, 64)
    with pytest.raises(ValueError):
        tp.shard_codes_k(torch.zeros(4, 64, dtype=torch.uint8), 32, 128)
