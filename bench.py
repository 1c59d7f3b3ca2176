"""Benchmark of the ternary BitLinear hot path on B200.

python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Workload ("decode_gemv_sweep"): the decode GEMV sweep at BitNet-2B-like shapes — projections
(N x K) 2560x2560, 6912x2560, 2560x6912, token batches M in {1, 4, 16, 64}, weights
N(0, 0.02) absmean-ternarized and packed 2 bits per weight, activations bf16 N(0,1) with
0.1 % outliers at +-20.  One step is one pass of the fused quantize-and-contract kernel over
a stack of independent layers of every (shape, M) pair (one grouped, persistent launch per
pair); the stacks hold more distinct packed weights (~0.6 GB) than the L2 cache, so every
launch streams its weights from HBM.  The per-pair breakdown also times the same stack as one
launch per layer, chained with programmatic dependent launch (the latency-bound form).
`value` is algorithmic GB/s (packed codes + scale + bf16 x + bf16 y per launch) over the whole
step with inputs resident in HBM; `e2e` is the same with the step's activations copied in from
pinned host memory and its outputs copied back inside the timed region (per stack, on three streams: copy-in,
launches and copy-out of consecutive stacks overlap).
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests", "golden"))

SHAPES = [(2560, 2560), (6912, 2560), (2560, 6912)]  # (N, K)
BATCHES = [1, 4, 16, 64]
# distinct weight matrices per shape: the count of each projection shape in one BitNet-2B-like model of 30 layers
# (4 attention-sized, 2 gate/up, 1 down per layer): 594 MB of packed weights
LAYERS = {(2560, 2560): 120, (6912, 2560): 60, (2560, 6912): 30}
METRIC = "ternary_decode_gemv_GBps"
GEMM_MIN_M = 16  # token batches from here on always run on the tensor-core contraction (one batched launch per layer stack);
                 # below it the library's measured rule decides per stack (ops.stack_uses_contraction: from 4 tokens on for K >= 4096)
REPEATS = 5      # the --steps region is timed this many times; the median is reported, with min and max
# DRAM bytes (ncu dram__bytes_read.sum + dram__bytes_write.sum of the streaming kernel's launches of the step, one
# capture of the bench command itself) over the algorithmic bytes of the same launch: (shape index, M) -> the ratio of
# the launch that holds the stack.  Stacks without a capture of their own use the mean of the measured ones.
NCU_TRAFFIC_RATIO = {(0, 1): 1.016, (1, 1): 1.016, (0, 4): 1.007, (1, 4): 1.007, (2, 1): 1.018, (2, 4): 1.018}


def algorithmic_bytes(m: int, n: int, k: int) -> int:
    """Packed codes + fp32 weight scale + bf16 activations read once + bf16 outputs."""
    return n * k // 4 + 4 + 2 * m * k + 2 * m * n


def reference_bytes(m: int, n: int, k: int) -> int:
    """The reference's own accounting (scripts/benchmark_kernels.py:61-66): int8 x, fp32 y."""
    return n * k // 4 + m * k + 4 * m * n


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            return json.load(f), "measured"
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}, "fallback"


class ClockSampler(threading.Thread):
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        super().__init__(daemon=True)
        self.index, self.samples, self.stop_flag, self.proc = index, [], False, None

    def run(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.Q}",
                                          "--format=csv,noheader,nounits", "-lms", "100"], stdout=subprocess.PIPE, text=True)
            for line in self.proc.stdout:
                if self.stop_flag:
                    break
                self.samples.append([c.strip() for c in line.split(",")])
        except OSError:
            pass

    def finish(self):
        self.stop_flag = True
        if self.proc is not None:
            self.proc.terminate()
        sm = [float(s[0]) for s in self.samples if s and s[0].replace(".", "").isdigit()]
        mx = [float(s[1]) for s in self.samples if len(s) > 1 and s[1].replace(".", "").isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = sorted({names[i] for s in self.samples if len(s) >= 6 for i in range(4) if s[2 + i].startswith("Active")})
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": reasons, "samples": len(sm)}


# ------------------------------------------------------------------ workload construction
def build_workload(wf, torch, device, rank: int, world: int, layers_scale: float = 1.0):
    """Packs the layer stacks on the device.  Returns a list of groups, one per (shape, M):
    dict(n, k, m, layers, x=[L, M, K'] bf16, y=[L, M, N'] bf16, group, reduce).

    With more than one rank the sweep is tensor-parallel the way the reference shards these projections:
    the 2560x2560 and 6912x2560 (q / gate / up like) matrices are column-parallel (rows split, no exchange),
    2560x6912 (down like) is row-parallel (K split at multiples of 64, one all-reduce of the partial outputs).
    Every rank builds the same full matrices (same seeds), ternarizes them whole and keeps its shard."""
    import inputs as gi

    if world > 1:
        from wrinklefree_monorepo_b200 import tp

    groups = []
    for si, (n, k) in enumerate(SHAPES):
        nl = max(2, int(LAYERS[(n, k)] * layers_scale))
        row_parallel = world > 1 and k > n
        g = torch.Generator(device="cpu").manual_seed(1000 * si)
        gd = torch.Generator(device=device).manual_seed(1000 * si)
        n_loc, k_lo, k_hi = n, 0, k
        if world > 1 and not row_parallel:
            r_lo, r_hi = tp.shard_bounds(n, world, 16)[rank]
            n_loc = r_hi - r_lo
        if row_parallel:
            k_lo, k_hi = tp.shard_bounds(k, world, 64)[rank]
        # the layers of a stack live in one contiguous buffer so that the batched contraction can walk them
        codes_stack = torch.empty(nl, n_loc, (k_hi - k_lo) // 4, dtype=torch.uint8, device=device)
        scales_stack = torch.empty(nl, 2, dtype=torch.float32, device=device)
        for li in range(nl):
            w = torch.randn(n, k, generator=gd, device=device, dtype=torch.float32) * 0.02
            codes, scale = wf.pack_ternary(w)  # one per-tensor scale for the whole matrix, then shard
            del w
            if world > 1 and not row_parallel:
                codes = tp.shard_codes_rows(codes, r_lo, r_hi)
            elif row_parallel:
                codes = tp.shard_codes_k(codes, k_lo, k_hi)
            codes_stack[li].copy_(codes)
            scales_stack[li].copy_(scale)
        lay = [(codes_stack[li], scales_stack[li]) for li in range(nl)]
        for m in BATCHES:
            x = torch.randn(nl, m, k, generator=g, dtype=torch.float32)
            x = gi.with_outliers(x, seed=1000 * si + m).to(torch.bfloat16)[..., k_lo:k_hi].contiguous()
            xd = x.to(device)
            y = torch.empty(nl, m, n_loc, dtype=torch.bfloat16, device=device)
            batched = m >= GEMM_MIN_M or (STACK_RULE and wf.stack_uses_contraction(m, k_hi - k_lo))
            grp = None if batched else wf.DecodeGroup([dict(x=xd[li], codes=c, w_scale=s, out=y[li]) for li, (c, s) in enumerate(lay)])
            # a workspace per contraction stack: the step quantizes the tokens of all of them before the first contraction
            ws = wf.prefill_workspace(nl * m, k_hi - k_lo, device) if batched else None
            groups.append(dict(n=n, k=k, m=m, layers=lay, x_host=x.pin_memory(), x=xd, y=y, group=grp, reduce=row_parallel,
                               batched=batched, codes_stack=codes_stack, scales_stack=scales_stack, ws=ws))
    # The stacks are independent.  Those on the tensor-core contraction go first: a contraction ends with a last wave of
    # tiles that leaves most SMs idle (600 tiles on 148 SMs are 4.05 waves), which the launch behind it fills -- the next
    # contraction, and behind the last one the first streaming launch, whose own tail is short (its CTAs claim small items
    # from a shared counter).  STREAMING_FIRST (--streaming-first) is the other order.
    groups.sort(key=lambda g_: g_["batched"] if STREAMING_FIRST else not g_["batched"])
    return groups


def merge_streaming(wf, groups):
    """The streaming stacks (M < GEMM_MIN_M) of equal K and equal M become ONE grouped launch each: the problems of a
    grouped launch need not be alike, and what a launch costs beside its bytes (entry to first data, the tail, the
    hand-over of the SMs to the next launch) is then paid once per launch instead of once per stack.
    Equal K because the shared-memory plan of a launch is made for its largest K (a 2560-wide stack inside a 6912-wide
    plan would keep half of its stages); equal M so that no weight matrix occurs twice in a launch: the M = 1 and M = 4
    stacks of a shape hold the same weights, and a launch over both found 39 % of its bytes in L2 (ncu: 569 MB of DRAM
    reads for 936 MB of algorithmic bytes), which is not the streaming case this bench is about."""
    by_key = {}
    for g in groups:
        if not g["batched"]:
            by_key.setdefault((g["k"], g["m"]), []).append(g)
    for members in by_key.values():
        if len(members) < 2:
            continue
        probs = [dict(x=m["x"][li], codes=c, w_scale=s_, out=m["y"][li]) for m in members for li, (c, s_) in enumerate(m["layers"])]
        merged = dict(members=members, group=wf.DecodeGroup(probs))
        for m in members:
            m["merged"] = merged


def run_group(wf, g, pdl: bool, reduce: bool = True):
    """One (shape, M) layer stack: one grouped launch (or the quantization + contraction pair for M >= GEMM_MIN_M)."""
    if g["batched"]:
        wf.bitlinear_batched(g["x"], g["codes_stack"], g["scales_stack"], out=g["y"])
    else:
        g["group"].run(pdl=pdl, x_ready=True)  # the stacks are independent: no launch writes the next one's x
    if reduce and g["reduce"]:  # row-parallel stack: sum the partial outputs of all ranks (the path's only exchange)
        import torch.distributed as dist

        dist.all_reduce(g["y"])


_SIDE = {}
STREAMING_FIRST = False
STACK_RULE = True  # --min-m-only: stacks below GEMM_MIN_M tokens all run on the streaming kernel
CHAIN_CONTRACTIONS = True  # --no-chain: every contraction stack quantizes in front of its own launch and waits for its predecessor


def run_step(wf, groups, pdl: bool):
    """One pass over the sweep (or over the given part of it): the streaming stacks whose merged launch is complete in
    `groups` run as that one launch, every other (shape, M) layer stack as its own grouped launch.  The exchange of a
    row-parallel stack runs on a second stream behind its launch: the stacks are independent, so the next stack's
    launches need not wait for it (the step ends when both streams have)."""
    import torch

    present = {id(g) for g in groups}
    done, launches = set(), 0
    main = torch.cuda.current_stream()
    side = None

    def exchange(members):
        nonlocal side
        members = [m for m in members if m["reduce"]]
        if not members:
            return
        import torch.distributed as dist

        if side is None:
            dev = torch.cuda.current_device()
            side = _SIDE.get(dev) or _SIDE.setdefault(dev, torch.cuda.Stream())
        side.wait_stream(main)
        with torch.cuda.stream(side):
            for m in members:
                dist.all_reduce(m["y"])

    # The contraction stacks: the tokens of all of them are quantized first (each stack into its own workspace), then
    # the contractions follow one another; all but the first are launched as independent of what runs ahead of them
    # (they are: own tokens, own workspace, own output), so each fills the SMs that the tail of its predecessor leaves.
    batched = [g for g in groups if g["batched"]]
    split = pdl and len(batched) > 1 and CHAIN_CONTRACTIONS
    if split:
        for g in batched:
            wf.prefill_quantize(g["x"], g["ws"], independent=True)
            launches += 1
    first = True
    for g in groups:
        mg = g.get("merged")
        if mg is not None and all(id(m) in present for m in mg["members"]):
            if id(mg) not in done:
                done.add(id(mg))
                mg["group"].run(pdl=pdl, x_ready=True)
                launches += 1
                exchange(mg["members"])
            continue
        if g["batched"] and split:
            wf.bitlinear_batched(g["x"], g["codes_stack"], g["scales_stack"], out=g["y"], workspace=g["ws"], quantized=True,
                                 independent=not first)
            first = False
            launches += 1
        else:
            run_group(wf, g, pdl, reduce=False)
            launches += 2 if g["batched"] else 1  # batched = quantization kernel + contraction
        exchange([g])
    if side is not None:
        main.wait_stream(side)
    return launches


def run_step_single(wf, groups, pdl: bool):
    """The same pass as one launch per layer (the dependent-chain form of a decoder)."""
    launches = 0
    for g in groups:
        x, y = g["x"], g["y"]
        for li, (codes, scale) in enumerate(g["layers"]):
            wf.bitlinear(x[li], codes, scale, out=y[li], pdl=pdl, path="decode")
            launches += 1
    return launches


def step_bytes(groups, fn=algorithmic_bytes) -> int:
    return sum(fn(g["m"], g["n"], g["k"]) * len(g["layers"]) for g in groups)


def capture(torch, fn):
    """Warm up on a side stream, then capture `fn` into a CUDA graph."""
    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(s):
        fn()
    torch.cuda.current_stream().wait_stream(s)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        fn()
    return graph


# ------------------------------------------------------------------ CPU reference arm
def host_threads() -> int:
    """Cores this process may use (a launcher may have exported OMP_NUM_THREADS=1: the thread count is set explicitly)."""
    try:
        return len(os.sched_getaffinity(0))
    except AttributeError:
        return os.cpu_count() or 1


def cpu_reference_run(steps: int, warmup: int, layers_scale: float = 1.0):
    """Times the reference's own CPU path on the sweep: per layer and token batch `quantize_activations_i8` of the fp32
    activations, then `bitnet_gemm_i2_i8` on I2_S weights (its bitnet_gemv.cpp compiled from its sources behind
    oracle/_ref, all host threads); falls back to the C port of the oracle when no compiled reference is present.
    The stacks have the benchmark's full layer counts; their weights are two random matrices per shape repeated through
    one contiguous buffer (distinct addresses, so the host caches see the same footprint as distinct layers)."""
    import numpy as np

    from oracle import bitlinear_oracle as O
    from oracle.clib import load_oracle, load_reference

    ref = load_reference()
    kind = "reference" if ref is not None else "port"
    port = load_oracle()
    cores = host_threads()
    if ref is not None:
        ref.set_num_threads(cores)
        cores = ref.num_threads()
    else:
        cores = port.num_threads()
    rng = np.random.default_rng(0)
    work = []
    for (n, k) in SHAPES:
        nl = max(2, int(LAYERS[(n, k)] * layers_scale))
        base = []
        for _ in range(2):  # N(0, 0.02) weights, absmean-ternarized
            w = (rng.standard_normal((n, k)) * 0.02).astype(np.float32)
            t = port.ternarize(w, port.absmean(w))
            base.append(O.pack_i2s(t) if ref is not None else port.pack_wf16(t))
        stack = np.empty((nl,) + base[0].shape, dtype=np.uint8)
        for li in range(nl):
            stack[li] = base[li % 2]
        for m in BATCHES:
            x = rng.standard_normal((m, k)).astype(np.float32)  # N(0, 1) with 0.1 % outliers at +-20, bf16 values
            out_mask = rng.random((m, k)) < 1e-3
            x = np.where(out_mask, np.where(rng.random((m, k)) < 0.5, -20.0, 20.0), x).astype(np.float32)
            work.append((n, k, m, stack, O.bf16_round(x)))

    def one_step():
        for (n, k, m, stack, x) in work:
            for li in range(stack.shape[0]):
                if ref is not None:
                    q, s = ref.quantize_activations(x)
                    ref.gemm(stack[li], q, 0.02 * float(s))
                else:
                    q, s = port.act_quant(x, 0)
                    port.gemm_wf16(q, stack[li])

    bytes_step = sum(algorithmic_bytes(m, n, k) * stack.shape[0] for (n, k, m, stack, _) in work)
    for _ in range(warmup):
        one_step()
    t0 = time.perf_counter()
    for _ in range(steps):
        one_step()
    dt = (time.perf_counter() - t0) / steps
    sample = (f"the full sweep ({[w[3].shape[0] for w in work[::len(BATCHES)]]} layers per shape x M in {BATCHES}), fp32 activations "
              f"quantized inside the timed loop, {steps} steps of {dt * 1e3:.1f} ms after {warmup} warm-up; kernel: " +
              ("quantize_activations_i8 + bitnet_gemm_i2_i8 (AVX-%s build of the reference's bitnet_gemv.cpp, OpenMP)" % ref.flavour.replace("avx", "")
               if ref is not None else "scalar C port of the oracle (OpenMP)"))
    return dict(value=bytes_step / dt / 1e9, unit="GB/s", cores=cores, kind=kind, sample=sample), steps, warmup, dt


def cpu_other_baselines():
    """The two other CPU paths the reference has for this operator, on a bounded sample (one layer per shape and token
    batch), same byte accounting: the PyTorch BitLinear forward (restated in oracle/torch_bitlinear.py: it re-ternarizes
    the fp32 weight on every call) and BitNet.cpp's ggml_vec_dot_i2_i8_s in an OpenMP row loop (oracle/_ref)."""
    import numpy as np
    import torch

    from oracle import bitlinear_oracle as O
    from oracle import torch_bitlinear as TB
    from oracle.clib import load_ggml_reference

    out = []
    cores = host_threads()
    torch.set_num_threads(cores)
    rng = np.random.default_rng(1)
    g = torch.Generator().manual_seed(1)
    for dt_name, dt in (("bf16", torch.bfloat16), ("f32", torch.float32)):
        tot_b, tot_t = 0, 0.0
        for (n, k) in [(1536, 576)] + SHAPES:
            w = torch.randn(n, k, generator=g) * 0.02
            for m in ([16] if (n, k) == (1536, 576) else BATCHES):
                x = torch.randn(m, k, generator=g).to(dt)
                with torch.no_grad():
                    TB.bitlinear_forward(x, w)
                    t0 = time.perf_counter()
                    TB.bitlinear_forward(x, w)
                    tot_t += time.perf_counter() - t0
                tot_b += algorithmic_bytes(m, n, k)
        out.append(dict(kind="port", path=f"PyTorch BitLinear.forward ({dt_name} input, weight re-ternarized per call)", cores=cores,
                        value=tot_b / tot_t / 1e9, unit="GB/s", sample="one layer per shape (config-1 shape and the three sweep shapes) and token batch"))
    gg = load_ggml_reference()
    if gg is not None:
        gg.set_num_threads(cores)
        tot_b, tot_t = 0, 0.0
        for (n, k) in SHAPES:
            if k % 128:
                continue
            packed = O.pack_i2s(rng.integers(-1, 2, size=(n, k)).astype(np.int8))
            for m in BATCHES:
                q = rng.integers(-127, 128, size=(m, k)).astype(np.int8)
                sums, scales = q.astype(np.int64).sum(1).astype(np.float32), np.full(m, 30.0, np.float32)
                gg.mul_mat(packed, q, sums, scales, 0.02)
                t0 = time.perf_counter()
                gg.mul_mat(packed, q, sums, scales, 0.02)
                tot_t += time.perf_counter() - t0
                tot_b += algorithmic_bytes(m, n, k)
        out.append(dict(kind="reference", path="BitNet.cpp ggml_vec_dot_i2_i8_s in an OpenMP row loop (AVX2 build of ggml-bitnet-mad.cpp)",
                        cores=gg.num_threads(), value=tot_b / tot_t / 1e9, unit="GB/s", sample="one layer per sweep shape and token batch, int8 activations given"))
    else:
        out.append(dict(kind="reference", path="BitNet.cpp ggml_vec_dot_i2_i8_s", unavailable="oracle/_ref holds no build of it on this host"))
    return out


# ------------------------------------------------------------------ prefill GEMM (secondary figures of the same line)
PREFILL_M = [512, 2048, 8192]


def int8_peak(wf):
    """Measured int8 tensor-core rate of this GPU (TOPS): every SM issues tcgen05.mma.kind::i8 M128 N256 K32 on operands
    resident in shared memory (the library's wf_probe_i8_mma); also the time per instruction at N = 16 and 64."""
    import ctypes as C

    lib = wf._lib.lib()
    res = {}
    for n in (256, 128, 64, 16):
        tops, ns = C.c_double(0), C.c_double(0)
        wf._lib.check(lib.wf_probe_i8_mma(n, 20000, C.byref(tops), C.byref(ns)), "wf_probe_i8_mma")
        res[n] = (tops.value, ns.value)
    return {"tops_n256": round(res[256][0], 1), "tops_n128": round(res[128][0], 1),
            "ns_per_mma": {str(n): round(res[n][1], 2) for n in res}}


def prefill_section(wf, torch, device, peak_tops, shapes=None, ms=None):
    """int8 x ternary GEMM on tcgen05 at the sweep's shapes: TOPS = 2*M*N*K / time, for the whole operator
    (activation quantization + contraction) with bf16 activations resident in HBM, and for the contraction alone on
    int8 activations.  Fractions: of the measured int8 rate (`peak_tops`, see int8_peak) and of the nominal 4500 TOPS."""
    out = []
    gd = torch.Generator(device=device).manual_seed(4242)
    for (n, k) in (shapes or [(2560, 2560), (6912, 2560), (2560, 6912)]):
        codes, scale = wf.pack_ternary(torch.randn(n, k, generator=gd, device=device) * 0.02)
        for m in (ms or PREFILL_M):
            x = torch.randn(m, k, generator=gd, device=device).to(torch.bfloat16)
            y = torch.empty(m, n, dtype=torch.bfloat16, device=device)
            xq, xs = wf.act_quant_i8(x)  # the reference's GEMM operator takes int8 activations and their scales

            def timed(fn):
                graph = capture(torch, fn)
                for _ in range(3):
                    graph.replay()
                torch.cuda.synchronize()
                a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                reps, samples = 10, []
                for _ in range(3):
                    a.record()
                    for _ in range(reps):
                        graph.replay()
                    b.record()
                    torch.cuda.synchronize()
                    samples.append(a.elapsed_time(b) * 1e3 / reps)
                return statistics.median(samples)

            us = timed(lambda: wf.bitlinear(x, codes, scale, out=y, path="prefill"))
            us_c = timed(lambda: wf.bitlinear(xq, codes, scale, x_scale=xs, out=y, path="prefill"))
            tops, tops_c = 2.0 * m * n * k / us / 1e6, 2.0 * m * n * k / us_c / 1e6
            out.append({"N": n, "K": k, "M": m, "us": round(us, 2), "TOPS": round(tops, 1),
                        "frac_of_measured_int8": round(tops / peak_tops, 4),
                        "frac_of_nominal_int8_4500": round(tops / 4500.0, 4),
                        "contraction_only": {"us": round(us_c, 2), "TOPS": round(tops_c, 1), "frac_of_measured_int8": round(tops_c / peak_tops, 4),
                                             "input": "int8 activations + per-token scales given (the operator signature of bitnet_gemm_i2_i8)"}})
    return out


# ------------------------------------------------------------------ the plug-in call, end to end
def plugin_e2e(wf, torch, device, steps: int, n: int = 2560, k: int = 2560, m: int = 16, nl: int = 120):
    """One stack of the sweep driven the way a serving framework drives the layer: per layer
    `BitNetLinearMethod.apply(layer, x)` on I2_S weights registered by `create_weights`, with that layer's activations
    copied from pinned host memory before the call and its fp32 output copied back after it, every step."""
    import inputs as gi

    method = wf.BitNetLinearMethod(wf.BitNetConfig())
    gd = torch.Generator(device=device).manual_seed(77)
    layers = []
    for _ in range(nl):
        codes, scale = wf.pack_ternary(torch.randn(n, k, generator=gd, device=device) * 0.02)
        layer = torch.nn.Module()
        method.create_weights(layer, k, [n], k, n, torch.bfloat16)
        layer = layer.to(device)
        layer.qweight.data.copy_(wf.repack(codes, wf._lib.LAYOUT_WF16, n, k, wf._lib.LAYOUT_I2S))
        layer.scale.data.copy_(scale[:1])
        method.process_weights_after_loading(layer)
        layers.append(layer)
    g = torch.Generator().manual_seed(78)
    x_host = gi.with_outliers(torch.randn(nl, m, k, generator=g), seed=78).to(torch.bfloat16).pin_memory()
    y_host = torch.empty(nl, m, n, dtype=torch.float32).pin_memory()
    x_dev = torch.empty(nl, m, k, dtype=torch.bfloat16, device=device)

    def step():
        for li, layer in enumerate(layers):
            x_dev[li].copy_(x_host[li], non_blocking=True)
            y_host[li].copy_(method.apply(layer, x_dev[li]), non_blocking=True)

    for _ in range(2):
        step()
    torch.cuda.synchronize()
    samples = []
    for _ in range(3):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(steps):
            step()
        b.record()
        torch.cuda.synchronize()
        samples.append(a.elapsed_time(b) / steps)
    ms = statistics.median(samples)
    return {"call": "BitNetLinearMethod.apply(layer, x) per layer, I2_S weights", "stack": f"{nl} layers of {n}x{k}, M = {m}",
            "ms_per_step": round(ms, 4), "us_per_layer": round(ms * 1e3 / nl, 3),
            "value": algorithmic_bytes(m, n, k) * nl / (ms * 1e-3) / 1e9, "unit": "GB/s",
            "h2d_bytes_per_step": x_host.numel() * 2, "d2h_bytes_per_step": y_host.numel() * 4}


# ------------------------------------------------------------------ tensor-parallel parity (multi-rank runs)
def tp_parity_check(wf, torch, dist, device, rank: int, world: int) -> str:
    """One small fixed case per rank, checked against the CPU oracle before anything is timed: the accumulators of
    this rank's column shard and of its row (K) shard bit for bit, the gathered column-parallel output and the reduced
    row-parallel output identical on all ranks, the peer-memory sum equal to the rank-ordered fp32 sum of the (oracle-
    checked) partial outputs, and one round of the peer-memory all-reduce against the library all-reduce.  The reduced
    output is also held to the UNSHARDED result within 2e-2 (max|a-b| / max|b|): every rank quantizes its K slice with
    its own per-token scale, as the reference's row-parallel layer does, so the two differ by the rounding noise of
    `world` independent quantizations (1.1e-2 at eight ranks of 512 inputs each) — a sanity bound, not the parity
    criterion.  Returns "ok" or the first failure; the oracle is the checker here, nothing of it is timed."""
    import numpy as np

    from oracle.clib import load_oracle
    from wrinklefree_monorepo_b200 import tp

    try:
        oc = load_oracle()
        n, k, m = 128 * world, 512 * world, 5
        g = torch.Generator().manual_seed(4321)
        w = torch.randn(n, k, generator=g) * 0.02
        x = torch.randn(m, k, generator=g).bfloat16()
        codes, scale = wf.pack_ternary(w.to(device))
        t = wf.unpack_codes(codes, n, k).cpu().numpy()
        s_w = float(scale[0])
        q_full, s_full = oc.act_quant(x.float().numpy(), 1)
        y_full = oc.rescale(oc.int_gemm(q_full, t), s_full, s_w)
        fails = []
        # column-parallel: rows of this rank
        col = tp.ColumnParallelBitLinear(codes, scale, k, n, gather_output=True)
        lo, hi = col.bounds[rank]
        _, acc = wf.bitlinear(x.to(device), col.codes, scale, want_acc=True, out_dtype=torch.float32)
        if not np.array_equal(acc.cpu().numpy(), oc.int_gemm(q_full, t[lo:hi])):
            fails.append("column shard accumulators differ from the oracle")
        yc = col(x.to(device), out_dtype=torch.float32)
        if not np.array_equal(yc.cpu().numpy(), y_full):
            fails.append("gathered column-parallel output differs from the oracle")
        # row-parallel: K slice of this rank, local activation scales
        row = tp.RowParallelBitLinear(codes, scale, k, n, reduce_dtype=torch.float32)
        k0, k1 = row.bounds[rank]
        x_loc = x[:, k0:k1].contiguous()
        q_loc, s_loc = oc.act_quant(x_loc.float().numpy(), 1)
        y_part, acc = wf.bitlinear(x_loc.to(device), row.codes, scale, want_acc=True, out_dtype=torch.float32)
        if not np.array_equal(acc.cpu().numpy(), oc.int_gemm(q_loc, t[:, k0:k1])):
            fails.append("row shard accumulators differ from the oracle")
        if not np.array_equal(y_part.cpu().numpy(), oc.rescale(oc.int_gemm(q_loc, t[:, k0:k1]), s_loc, s_w)):
            fails.append("row shard partial output differs from the oracle")
        parts = [torch.empty_like(y_part) for _ in range(world)]
        dist.all_gather(parts, y_part)
        want = parts[0].clone()
        for p_ in parts[1:]:
            want += p_  # fixed rank order, fp32
        yr = row(x_loc.to(device), out_dtype=torch.float32)  # library all-reduce
        err = float((yr.cpu() - torch.from_numpy(y_full)).abs().max() / np.abs(y_full).max())
        if err > 2e-2:
            fails.append(f"reduced row-parallel output off the unsharded result by {err:.3e}")
        one = tp.OneShotAllReduce()
        row2 = tp.RowParallelBitLinear(codes, scale, k, n, reduce_dtype=torch.float32, all_reduce=one)
        yo = row2(x_loc.to(device), out_dtype=torch.float32)
        if one._ctx is not None and not torch.equal(yo, want):
            fails.append("peer-memory all-reduce differs from the rank-ordered fp32 sum")
        for name, y_ in (("library", yr), ("peer-memory", yo)):
            allr = [torch.empty_like(y_) for _ in range(world)]
            dist.all_gather(allr, y_)
            if any(not torch.equal(allr[0], a_) for a_ in allr[1:]):
                fails.append(f"{name} all-reduce: ranks hold different bits")
        b = torch.randn(64, 4096, generator=torch.Generator().manual_seed(rank)).bfloat16().to(device)
        b1, b2 = b.clone(), b.clone()
        one(b1)
        dist.all_reduce(b2)
        if float((b1.float() - b2.float()).abs().max()) > 2e-2 * float(b2.float().abs().max()):
            fails.append("peer-memory all-reduce (bf16) off the library all-reduce")
        one.status()
        ok = torch.tensor([0 if fails else 1], device=device)
        dist.all_reduce(ok, op=dist.ReduceOp.MIN)
        if fails:
            return f"rank {rank}: " + "; ".join(fails)
        return "ok" if int(ok.item()) == 1 else "a rank other than 0 failed (see its stderr)"
    except Exception as e:  # the benchmark line must still be printed
        return "error: " + repr(e)[:300]


# ------------------------------------------------------------------ decoder tokens/s (secondary figures)
def decoder_section(wf, torch, device, world, full: bool):
    """Greedy decode tokens/s of random-init ternary decoders on the BitLinear kernels (CUDA-graphed step):
    Llama-3-8B shape at a 2048-token context for batch 1, 32 and 256 (--decoder-quick drops 256), tensor-parallel over
    the ranks; on one GPU also the SmolLM2-135M shape (batch 32, 512-token prompt, 128 steps)."""
    from wrinklefree_monorepo_b200.decoder import LLAMA3_8B, SMOLLM2_135M, TernaryDecoder

    out = []

    def timed(model, steps):
        model.graph.replay()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(steps):
            model.graph.replay()
            model.tok.copy_(model.next_tok)
        b.record()
        torch.cuda.synchronize()
        return a.elapsed_time(b) / steps

    for batch in ([1, 32, 256] if full else [1, 32]):
        model = TernaryDecoder(LLAMA3_8B, batch, 2048 + 32, device, seed=7)  # room for the timed steps behind the context
        for L in model.layers:  # a context of 2048 random tokens' keys and values
            L["kc"].normal_()
            L["vc"].normal_()
        model.pos.fill_(2047)
        model.capture(masked=False)
        ms = timed(model, 16)
        by = model.weight_bytes_per_step()
        row = {"model": "llama3-8b-shape", "tp": world, "batch": batch, "context": 2048, "ms_per_step": round(ms, 3),
               "tok_s": round(batch / ms * 1e3, 1), "GB_per_step_per_rank": round(by / 1e9, 3),
               "GBps_per_rank": round(by / ms / 1e6, 1), "attention": "wf_attn_decode_bf16"}
        if world == 1:  # the same step with the framework's fused attention in place of this library's kernel
            model.pos.fill_(2047)
            model.capture(masked=False, attention="library")
            row["ms_per_step_library_attention"] = round(timed(model, 16), 3)
        out.append(row)
        del model
        torch.cuda.empty_cache()
    if world == 1:
        model = TernaryDecoder(SMOLLM2_135M, 32, 512 + 160, device, seed=8)
        g = torch.Generator().manual_seed(9)
        ids = torch.randint(0, SMOLLM2_135M.vocab, (32, 512), generator=g).to(device)
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        model.prefill(ids)
        torch.cuda.synchronize()
        t_prefill = time.perf_counter() - t0
        model.capture(masked=True)
        ms = timed(model, 128)
        out.append({"model": "smollm2-135m-shape", "tp": 1, "batch": 32, "prompt": 512, "decode_steps": 128,
                    "prefill_ms": round(t_prefill * 1e3, 1), "ms_per_step": round(ms, 3), "tok_s": round(32 / ms * 1e3, 1)})
    return out


def step_kernels_section(wf, torch, device):
    """The two kernels of the decode step that are not BitLinear, timed alone on the 8B shape (CUDA graph of four calls on
    distinct tensors, median of three): the bf16 output head (128,256 x 4096, read once per token batch) and the decode
    attention over a 2048-token bf16 KV cache (32 query / 8 KV heads of 128), with their algorithmic GB/s."""
    hbm = measured_peaks()[0]["hbm_gbs"]
    out = {"output_head": [], "decode_attention": []}

    def timed(fn):
        graph = capture(torch, fn)
        for _ in range(2):
            graph.replay()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        samples = []
        for _ in range(3):
            a.record()
            for _ in range(5):
                graph.replay()
            b.record()
            torch.cuda.synchronize()
            samples.append(a.elapsed_time(b) * 1e3 / 5)
        return statistics.median(samples)

    vocab, hidden = 128256, 4096
    g = torch.Generator(device=device).manual_seed(11)
    heads = [(torch.randn(vocab, hidden, generator=g, device=device) * 0.02).bfloat16() for _ in range(2)]  # 2.1 GB: larger than L2
    for batch in (1, 32, 256):
        x = torch.randn(batch, hidden, generator=g, device=device).bfloat16()
        y = torch.empty(batch, vocab, dtype=torch.bfloat16, device=device)
        us = timed(lambda: [wf.linear_bf16(x, w_, out=y) for w_ in heads]) / len(heads)
        byts = vocab * hidden * 2 + batch * hidden * 2 + batch * vocab * 2
        out["output_head"].append({"batch": batch, "us": round(us, 1), "GBps": round(byts / us / 1e3, 1), "frac_hbm": round(byts / us / 1e3 / hbm, 4)})
    del heads
    torch.cuda.empty_cache()
    nq, nkv, d, t = 32, 8, 128, 2048 + 32
    for batch in (1, 32, 256):
        n = 4 if batch < 256 else 2  # distinct caches, so that a small batch does not sit in L2
        q = torch.randn(batch, nq * d, generator=g, device=device).bfloat16()
        caches = [(torch.randn(batch, nkv, t, d, generator=g, device=device).bfloat16(), torch.randn(batch, nkv, t, d, generator=g, device=device).bfloat16())
                  for _ in range(n)]
        o = torch.empty(batch, nq * d, dtype=torch.bfloat16, device=device)
        pos = torch.tensor(2047, dtype=torch.long, device=device)
        us = timed(lambda: [wf.ops.attn_decode(q, kc, vc, pos, o) for kc, vc in caches]) / n
        byts = 2 * batch * nkv * 2048 * d * 2
        out["decode_attention"].append({"batch": batch, "context": 2048, "us": round(us, 1), "GBps": round(byts / us / 1e3, 1),
                                        "frac_hbm": round(byts / us / 1e3 / hbm, 4)})
        del caches
        torch.cuda.empty_cache()
    return out


# ------------------------------------------------------------------ main
def finish(dist, torch, rank):
    """Multi-rank exit.  The CUDA graphs of this run captured NCCL kernels, and tearing a communicator down while
    such graphs exist blocks; every rank has nothing left to do after the final barrier, so the processes leave
    without the teardown (exit status 0)."""
    dist.barrier()
    torch.cuda.synchronize()
    note(rank, "final barrier passed")
    sys.stdout.flush()
    sys.stderr.flush()
    os._exit(0)


def note(rank, msg):
    """Progress marker on stderr (one line per phase and rank)."""
    print(f"[bench r{rank} {time.strftime('%H:%M:%S')}] {msg}", file=sys.stderr, flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--layers-scale", type=float, default=1.0, help="scale the layer stacks (profiling on a small case)")
    ap.add_argument("--no-pdl", action="store_true")
    ap.add_argument("--prefill-only", action="store_true", help="run only the prefill GEMM section (profiling)")
    ap.add_argument("--no-decoder", action="store_true", help="skip the decoder tokens/s section")
    ap.add_argument("--decoder-only", action="store_true", help="run only the decoder tokens/s section (profiling)")
    ap.add_argument("--decoder-quick", action="store_true", help="skip batch 256 of the 8B shape")
    ap.add_argument("--kernels-only", action="store_true", help="run only the output-head / decode-attention timings (profiling)")
    ap.add_argument("--only-m", type=int, default=0, help="restrict the sweep to one token batch (profiling)")
    ap.add_argument("--only-shape", type=int, default=-1, help="restrict the sweep to one shape index (profiling)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--streaming-first", action="store_true", help="the streaming launches of a step before its contractions (ablation of the order)")
    ap.add_argument("--min-m-only", action="store_true", help="every stack below 16 tokens on the streaming kernel (ablation of the dispatch rule)")
    ap.add_argument("--no-chain", action="store_true", help="contraction stacks as quantization + launch pairs that wait for one another")
    ap.add_argument("--no-merge", action="store_true", help="one grouped launch per (shape, M) stack instead of one per (K, M)")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    warmup = max(args.warmup, 3)
    config = {"workload": "decode_gemv_sweep", "shapes_NxK": ["%dx%d" % s for s in SHAPES], "batches_M": BATCHES,
              "layers_per_shape": [max(2, int(LAYERS[s] * args.layers_scale)) for s in SHAPES], "activations": "bf16 N(0,1) + 0.1% outliers at +-20",
              "weights": "N(0,0.02) absmean-ternarized, 2 bits/weight", "l2": "inputs larger than L2 (distinct weights per launch)"}

    if args.impl == "reference":
        if rank != 0:
            return
        cb, steps, wu, dt = cpu_reference_run(args.steps, warmup, args.layers_scale)
        line = {"impl": "reference", "metric": METRIC, "value": cb["value"], "unit": "GB/s", "n_gpus": args.gpus,
                "steps": steps, "warmup": wu, "ms_per_step": dt * 1e3, "higher_is_better": True, "scaling": "strong",
                "vs_baseline": None, "dtype": "u8xs8->s32", "data": "synthetic", "config": config, "cpu_baseline": cb,
                "e2e": {"value": cb["value"], "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
                "gpu_launches": 0}
        print(json.dumps(line))
        return

    import torch

    from __graft_entry__ import load_package

    wf = load_package()
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    if not wf.check_kernel_available():
        raise RuntimeError("wf_b200 library / sm_100 device unavailable: " + wf._lib.lib().wf_last_error().decode())
    dist = None
    if world > 1:
        import torch.distributed as dist

        import datetime

        # NCCL announces its version on stdout when the communicator comes up; stdout carries the one JSON line only
        saved = os.dup(1)
        os.dup2(2, 1)
        try:
            dist.init_process_group("nccl", device_id=device, timeout=datetime.timedelta(seconds=90))
            dist.barrier()
            torch.cuda.synchronize()
        finally:
            sys.stdout.flush()
            os.dup2(saved, 1)
            os.close(saved)

    if args.decoder_only:
        res = decoder_section(wf, torch, device, world, not args.decoder_quick)
        if rank == 0:
            print(json.dumps({"decode_tok_s": res}))
        return
    if args.kernels_only:
        print(json.dumps({"step_kernels": step_kernels_section(wf, torch, device)}))
        return
    if args.prefill_only:
        peaks, _ = measured_peaks()
        res = prefill_section(wf, torch, device, int8_peak(wf)["tops_n256"], [SHAPES[args.only_shape]] if args.only_shape >= 0 else None,
                              [args.only_m] if args.only_m else None)
        print(json.dumps({"prefill_gemm": res}))
        return
    if args.only_m:
        BATCHES[:] = [args.only_m]
    if args.only_shape >= 0:
        SHAPES[:] = [SHAPES[args.only_shape]]
    if args.min_m_only:
        global STACK_RULE
        STACK_RULE = False
    if args.streaming_first:
        global STREAMING_FIRST
        STREAMING_FIRST = True
    note(rank, "building workload")
    groups = build_workload(wf, torch, device, rank, world, args.layers_scale)
    if args.no_chain:
        global CHAIN_CONTRACTIONS
        CHAIN_CONTRACTIONS = False
    if not args.no_merge:
        merge_streaming(wf, groups)
    note(rank, "capturing step graph")
    pdl = not args.no_pdl
    counted = {}
    try:
        graph = capture(torch, lambda: counted.__setitem__("n", run_step(wf, groups, pdl)))
    except RuntimeError as e:  # programmatic dependent launch not capturable here: plain edges
        if not pdl:
            raise
        print(f"[bench] capture with programmatic dependent launch failed ({e}); retrying without", file=sys.stderr)
        pdl = False
        torch.cuda.synchronize()
        graph = capture(torch, lambda: counted.__setitem__("n", run_step(wf, groups, pdl)))
    launches = counted["n"]  # kernels of this library per step
    total_bytes = step_bytes(groups)

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- tensor-parallel parity evidence (every rank, before anything is timed)
    tp_parity = None
    if dist is not None:
        note(rank, "tensor-parallel parity check")
        tp_parity = tp_parity_check(wf, torch, dist, device, rank, world)

    def timed_replays(gr, steps):
        """REPEATS timings of `steps` replays each, on the device, max over ranks per repeat -> list of ms per step."""
        out = []
        for _ in range(REPEATS):
            barrier()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            for _ in range(steps):
                gr.replay()
            b.record()
            barrier()
            out.append(a.elapsed_time(b) / steps)
        if dist is not None:
            t = torch.tensor(out, device=device)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            out = t.tolist()
        return out

    note(rank, "device-resident timing")
    for _ in range(warmup):
        graph.replay()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
        time.sleep(0.3)
    ms_all = timed_replays(graph, args.steps)
    ms = statistics.median(ms_all)

    note(rank, "end-to-end timing")
    # ---- end to end: pinned host activations in, outputs back to pinned host memory, every step
    h2d = sum(g["x_host"].numel() * 2 for g in groups)
    d2h = sum(g["y"].numel() * 2 for g in groups)
    y_host = [torch.empty(g["y"].shape, dtype=torch.bfloat16).pin_memory() for g in groups]

    # Three streams: the copy-in of stack g, the launches of stack g - 1 and the copy-out of stack g - 2 overlap
    # (the two copy directions run at the same time on the link); events order them per stack, also from one
    # step to the next (x is not overwritten before the launch that read it has finished, y not before it is out).
    s_in, s_run, s_out = torch.cuda.Stream(), torch.cuda.Stream(), torch.cuda.Stream()
    ev_in = [torch.cuda.Event() for _ in groups]
    ev_run = [torch.cuda.Event() for _ in groups]
    ev_out = [torch.cuda.Event() for _ in groups]
    state = {"first": True}

    def e2e_fork():
        for s_ in (s_in, s_run, s_out):
            s_.wait_stream(torch.cuda.current_stream())

    def e2e_join():
        for s_ in (s_in, s_run, s_out):
            torch.cuda.current_stream().wait_stream(s_)

    # order of the stacks in the pipeline: the first copy-in and the last copy-out overlap with nothing, so the two
    # smallest stacks go to the ends and the large ones to the middle
    # (sizes of the unsharded stacks: every rank must walk the stacks in the same order, some carry an all-reduce)
    by_size = sorted(range(len(groups)), key=lambda i_: (groups[i_]["m"] * (groups[i_]["n"] + groups[i_]["k"]) * len(groups[i_]["layers"]), i_))
    e2e_order = by_size[:1] + by_size[2:][::-1] + by_size[1:2] if len(by_size) > 2 else by_size

    def e2e_step():
        for i in e2e_order:
            g, yh = groups[i], y_host[i]
            with torch.cuda.stream(s_in):
                if not state["first"]:
                    s_in.wait_event(ev_run[i])  # last step's launch has read x
                g["x"].copy_(g["x_host"], non_blocking=True)
                ev_in[i].record(s_in)
            with torch.cuda.stream(s_run):
                s_run.wait_event(ev_in[i])
                if not state["first"]:
                    s_run.wait_event(ev_out[i])  # last step's y has been copied out
                run_group(wf, g, False)
                ev_run[i].record(s_run)
            with torch.cuda.stream(s_out):
                s_out.wait_event(ev_run[i])
                yh.copy_(g["y"], non_blocking=True)
                ev_out[i].record(s_out)
        state["first"] = False

    e2e_fork()
    for _ in range(3):
        e2e_step()
    e2e_join()
    e2e_all = []
    for _ in range(REPEATS):
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        e2e_fork()
        for _ in range(args.steps):
            e2e_step()
        e2e_join()
        e1.record()
        barrier()
        e2e_all.append(e0.elapsed_time(e1) / args.steps)
    if dist is not None:
        t = torch.tensor(e2e_all, device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_all = t.tolist()
    ms_e2e = statistics.median(e2e_all)
    clocks = sampler.finish() if rank == 0 else None

    # ---- the same through the plug-in call a serving framework makes (one stack, one GPU): per layer
    # BitNetLinearMethod.apply(layer, x) on I2_S weights, host activations in, fp32 outputs back, every step
    plugin = plugin_e2e(wf, torch, device, args.steps) if (world == 1 and not args.only_m and args.only_shape < 0) else None

    peaks, peak_kind = measured_peaks()
    # the whole (unsharded) sweep's algorithmic bytes over the slowest rank's time
    full_bytes = sum(algorithmic_bytes(g["m"], g["n"], g["k"]) * len(g["layers"]) for g in groups)
    value = full_bytes / (ms * 1e-3) / 1e9
    # roofline of the HBM-bound kernel of the path (the fused quantize + GEMV decode kernel): its launches of the step
    # (the M < GEMM_MIN_M groups), timed on their own with CUDA events; the M >= GEMM_MIN_M groups run on the tensor-core
    # contraction and are reported under "roofline_gemm"
    dec_groups = [g for g in groups if not g["batched"]]
    gemm_groups = [g for g in groups if g["batched"]]

    def time_groups(gs):
        if not gs:
            return None
        gr = capture(torch, lambda: counted.__setitem__(id(gs), run_step(wf, gs, pdl)))
        for _ in range(3):
            gr.replay()
        return statistics.median(timed_replays(gr, args.steps))

    note(rank, "timing kernel families")
    ms_dec, ms_gemm = time_groups(dec_groups), time_groups(gemm_groups)
    note(rank, "breakdown")
    gemm_ops = sum(2.0 * g["m"] * g["n"] * g["k"] * len(g["layers"]) for g in gemm_groups)
    n_gemm_groups = len(gemm_groups)
    dec_names = ", ".join(f"{g_['n']}x{g_['k']} M={g_['m']}" for g_ in dec_groups)  # (the groups are emptied before the decoder section)
    gemm_names = ", ".join(f"{g_['n']}x{g_['k']} M={g_['m']}" for g_ in gemm_groups)
    dec_launches = max(1, counted.get(id(dec_groups), len(dec_groups)))
    per_launch_bytes = step_bytes(dec_groups) / dec_launches / world if dec_groups else 0.0  # what one rank's kernel moves
    per_launch_us = (ms_dec or 0.0) * 1e3 / dec_launches
    achieved = per_launch_bytes / (per_launch_us * 1e-6) / 1e9 if dec_groups else 0.0
    # DRAM traffic per launch from the ncu captures of these stacks (ratio to the algorithmic bytes, per stack)
    mean_ratio = sum(NCU_TRAFFIC_RATIO.values()) / len(NCU_TRAFFIC_RATIO)
    shape_idx = {s_: i_ for i_, s_ in enumerate([(2560, 2560), (6912, 2560), (2560, 6912)])}
    traffic = sum(algorithmic_bytes(g["m"], g["n"], g["k"]) * len(g["layers"]) / world *
                  NCU_TRAFFIC_RATIO.get((shape_idx.get((g["n"], g["k"]), -1), g["m"]), mean_ratio) for g in dec_groups) / dec_launches
    # per (shape, M) breakdown, each group timed alone over its own layer stack (every rank takes part: the
    # row-parallel groups contain the all-reduce)
    breakdown = []
    for g in groups:
        gg = [g]
        gr = capture(torch, lambda: run_step(wf, gg, pdl))
        for _ in range(3):
            gr.replay()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        reps, samples = 10, []
        for _ in range(3):
            a.record()
            for _ in range(reps):
                gr.replay()
            b.record()
            torch.cuda.synchronize()
            samples.append(a.elapsed_time(b) * 1e3 / reps / len(g["layers"]))
        us = statistics.median(samples)
        # the same stack as one launch per layer, chained with programmatic dependent launch
        gs = capture(torch, lambda: run_step_single(wf, gg, pdl))
        for _ in range(3):
            gs.replay()
        torch.cuda.synchronize()
        a.record()
        for _ in range(reps):
            gs.replay()
        b.record()
        torch.cuda.synchronize()
        us_single = a.elapsed_time(b) * 1e3 / reps / len(g["layers"])
        by = algorithmic_bytes(g["m"], g["n"], g["k"])
        breakdown.append({"N": g["n"], "K": g["k"], "M": g["m"], "layers": len(g["layers"]),
                          "kernel": "prefill_kernel" if g["batched"] else "decode_stream_kernel",
                          "us_per_layer_grouped": round(us, 3), "GBps": round(by / us / 1e3, 1),
                          "frac_hbm": round(by / us / 1e3 / peaks["hbm_gbs"], 4),
                          "GBps_reference_accounting": round(reference_bytes(g["m"], g["n"], g["k"]) / us / 1e3, 1),
                          "us_per_launch_single_chain": round(us_single, 3)})
    decoder = None
    if not args.no_decoder and not args.only_m and args.only_shape < 0:
        graph = None
        for g in groups:  # free the sweep's buffers first
            g.clear()
        torch.cuda.empty_cache()
        note(rank, "decoder section")
        try:
            decoder = decoder_section(wf, torch, device, world, not args.decoder_quick)
        except Exception as e:  # the main line must survive a failure of this secondary section
            decoder = [{"error": repr(e)[:300]}]
    note(rank, "done with collective phases")
    if rank != 0:
        # stay in step with rank 0 (it still runs single-GPU sections): tear the group down together
        finish(dist, torch, rank)
        return
    med = lambda v: {"median": round(statistics.median(v), 5), "min": round(min(v), 5), "max": round(max(v), 5), "repeats": len(v)}
    line = {"metric": METRIC, "value": value, "unit": "GB/s", "n_gpus": world, "steps": args.steps, "warmup": warmup,
            "ms_per_step": ms, "ms_per_step_repeats": med(ms_all), "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": "u8xs8->s32", "data": "synthetic", "config": config,
            "launch": {"pdl": pdl, "graph": True, "parallelism": f"tp{world}" if world > 1 else "single",
                       "streaming_kernel_stacks": dec_names, "contraction_stacks": gemm_names,
                       "contractions_chained": bool(pdl and CHAIN_CONTRACTIONS and n_gemm_groups > 1),
                       "streaming_stacks_merged_by_K_and_M": not args.no_merge},
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                         "frac": achieved / peaks["hbm_gbs"], "frac_of_nominal_8000": achieved / 8000.0, "traffic": traffic,
                         "traffic_source": "ncu dram__bytes_read.sum + dram__bytes_write.sum of the step's streaming launches, as a ratio to the "
                                           "algorithmic bytes: " + ", ".join(f"shape {k_[0]} M={k_[1]}: {v_:.3f}" for k_, v_ in sorted(NCU_TRAFFIC_RATIO.items())) +
                                           "; other stacks: their mean",
                         "peak_kind": peak_kind + " copy bandwidth",
                         "kernel": "decode_stream_kernel", "launches": f"the {dec_launches} grouped launches of the step that hold its {len(dec_groups)} stacks on the streaming kernel: " + dec_names
                                     + (" (stacks of equal K and M share a launch)" if dec_launches < len(dec_groups) else ""),
                         "bytes_per_launch": per_launch_bytes, "us_per_launch": per_launch_us},
            "e2e": {"value": full_bytes / (ms_e2e * 1e-3) / 1e9, "unit": "GB/s", "h2d_bytes_per_step": h2d,
                    "d2h_bytes_per_step": d2h, "ms_per_step": ms_e2e, "ms_per_step_repeats": med(e2e_all),
                    "call": "ops.DecodeGroup.run / ops.bitlinear_batched per stack (ctypes -> C ABI), pinned host buffers, three streams"},
            "gpu_launches": launches * args.steps, "clocks": clocks, "breakdown": breakdown}
    if plugin is not None:
        line["e2e"]["plugin"] = plugin
    if tp_parity is not None:
        line["tp_parity"] = tp_parity
    i8 = None
    if world == 1 or rank == 0:
        try:
            i8 = int8_peak(wf)
            line["int8_peak_measured"] = i8
        except Exception as e:
            line["int8_peak_measured"] = {"error": repr(e)[:200]}
    peak_tops = i8["tops_n256"] if i8 else 4500.0
    if n_gemm_groups and ms_gemm:
        tops = gemm_ops / (ms_gemm * 1e-3) / 1e12
        line["roofline_gemm"] = {"bound": "tensor", "kernel": "prefill_kernel (batched over each layer stack)",
                                 "launches": f"the {n_gemm_groups} stacks on the contraction: " + gemm_names, "achieved": tops,
                                 "unit": "TOPS", "peak": peak_tops,
                                 "peak_kind": "measured tcgen05.mma.kind::i8 rate (M128 N256 K32, operands resident)" if i8 else "nominal",
                                 "frac": tops / peak_tops, "frac_of_nominal_4500": tops / 4500.0, "ms": ms_gemm,
                                 "note": "useful ops 2*M*N*K; at M = 16 / 64 these stacks are bound by weight streaming and the "
                                         "expansion of the packed weights, not by the tensor rate"}
    if decoder is not None:
        line["decode_tok_s"] = decoder
        if world == 1:
            try:
                line["step_kernels"] = step_kernels_section(wf, torch, device)
            except Exception as e:  # a secondary figure must not cost the line
                line["step_kernels"] = {"error": repr(e)[:200]}
    if not args.only_m and args.only_shape < 0:
        note(rank, "prefill GEMM section")
        line["prefill_gemm"] = prefill_section(wf, torch, device, peak_tops)
        note(rank, "prefill GEMM section done")
    if not args.no_cpu_baseline and world == 1:
        cb, _, _, _ = cpu_reference_run(3, 1, args.layers_scale)
        try:
            cb["others"] = cpu_other_baselines()
        except Exception as e:
            cb["others"] = [{"error": repr(e)[:200]}]
        line["cpu_baseline"] = cb
    print(json.dumps(line), flush=True)
    if dist is not None:
        finish(dist, torch, rank)


if __name__ == "__main__":
    main()
