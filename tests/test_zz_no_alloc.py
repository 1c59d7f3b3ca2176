"""The allocation-free packing entry point, called through the C ABI.

wf_pack_ternary_noalloc exists for hosts that may not allocate device memory where they pack weights
(a serving process whose pool owns the GPU, a thread that cannot take cudaMalloc's implicit
synchronisation): its scratch is a fixed array inside the library.  The test packs the same matrices with
it and with wf_pack_ternary (caller scratch) and requires identical bytes and scales, twice in a row,
because consecutive calls reuse the same array.  This file sorts last on purpose: a run that stops at
the first failure has then already run every other test.
"""
import ctypes as C

import numpy as np
import pytest
import torch

DEV = "cuda:0"


def _both(wf, w, mode):
    lib = wf._lib.lib()
    n, k = w.shape
    dt = {torch.float32: 0, torch.float16: 1, torch.bfloat16: 2}[w.dtype]
    stream = torch.cuda.current_stream().cuda_stream
    codes_a = torch.empty(n, k // 4, dtype=torch.uint8, device=DEV)
    scale_a = torch.empty(2, dtype=torch.float32, device=DEV)
    scratch = torch.empty(max(8, lib.wf_pack_scratch_bytes(n, k)), dtype=torch.uint8, device=DEV)
    wf._lib.check(lib.wf_pack_ternary(w.data_ptr(), dt, n, k, w.stride(0), mode, 1e-5, codes_a.data_ptr(), scale_a.data_ptr(),
                                      scratch.data_ptr(), scratch.numel(), stream), "wf_pack_ternary")
    codes_b = torch.empty_like(codes_a)
    scale_b = torch.empty_like(scale_a)
    wf._lib.check(lib.wf_pack_ternary_noalloc(w.data_ptr(), dt, n, k, w.stride(0), mode, 1e-5, codes_b.data_ptr(),
                                              scale_b.data_ptr(), stream), "wf_pack_ternary_noalloc")
    return (codes_a, scale_a), (codes_b, scale_b)


@pytest.mark.gpu
def test_noalloc_pack_matches_regular_entry_point_twice(wf):
    assert wf._lib.lib().wf_pack_noalloc_scratch_bytes() == 148 * 8 * 8
    g = torch.Generator().manual_seed(99)
    first = torch.randn(1536, 576, generator=g) * 0.02      # BASELINE config 1 shape
    second = torch.randn(2560, 6912, generator=g) * 0.05    # a larger matrix, other scale: stale partial sums would show
    for call, (w, mode) in enumerate(((first, 0), (second, 0), (first.bfloat16(), 1), (first, 0))):
        (ca, sa), (cb, sb) = _both(wf, w.to(DEV), mode)
        torch.cuda.synchronize()
        assert torch.equal(ca, cb), f"codes differ on call {call}"
        assert torch.equal(sa, sb), f"scales differ on call {call}"
    # and against the oracle once, so the comparison is not between two equal mistakes
    from oracle import bitlinear_oracle as O

    (ca, sa), (cb, sb) = _both(wf, first.to(DEV), 0)
    t, s = O.ternarize_absmean(first.numpy())
    assert np.array_equal(cb.cpu().numpy(), O.pack_wf16(t)) and sb[0].item() == s


def test_noalloc_pack_rejects_oversized_matrices(wf):
    """The size limit is checked before anything touches a device, so this needs no GPU."""
    lib = wf._lib.lib()
    buf = (C.c_char * 4096)()
    p = (C.addressof(buf) + 255) // 256 * 256
    rc = lib.wf_pack_ternary_noalloc(p, 0, 1 << 15, 1 << 14, 1 << 14, 0, 1e-5, p, p, None)  # 2^29 weights
    assert rc == 4 and b"exceed the maximum" in lib.wf_last_error()
    rc = lib.wf_pack_ternary_noalloc(None, 0, 64, 64, 64, 0, 1e-5, p, p, None)
    assert rc == 1
