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
GEMM_MIN_M = 16  # token batches from here on run on the tensor-core contraction (one batched launch per layer stack)
NCU_TRAFFIC_RATIO = 203.52 / 197.84  # dram bytes / algorithmic bytes, profiles/decode_stream_kernel_m1_2560x2560.md


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
            batched = m >= GEMM_MIN_M
            grp = None if batched else wf.DecodeGroup([dict(x=xd[li], codes=c, w_scale=s, out=y[li]) for li, (c, s) in enumerate(lay)])
            groups.append(dict(n=n, k=k, m=m, layers=lay, x_host=x.pin_memory(), x=xd, y=y, group=grp, reduce=row_parallel,
                               batched=batched, codes_stack=codes_stack, scales_stack=scales_stack))
    # the stacks are independent: those on the streaming kernel go first, so that their launches chain (each starts
    # while its predecessor drains), then those on the tensor-core contraction
    groups.sort(key=lambda g_: g_["batched"])
    return groups


def run_group(wf, g, pdl: bool):
    """One (shape, M) layer stack: one grouped launch (or the quantization + contraction pair for M >= GEMM_MIN_M)."""
    if g["batched"]:
        wf.bitlinear_batched(g["x"], g["codes_stack"], g["scales_stack"], out=g["y"])
    else:
        g["group"].run(pdl=pdl, x_ready=True)  # the stacks are independent: no launch writes the next one's x
    if g["reduce"]:  # row-parallel stack: sum the partial outputs of all ranks (the path's only exchange)
        import torch.distributed as dist

        dist.all_reduce(g["y"])


def run_step(wf, groups, pdl: bool):
    """One pass over the sweep: every (shape, M) layer stack is one grouped launch."""
    for g in groups:
        run_group(wf, g, pdl)
    return sum(2 if g["batched"] else 1 for g in groups)  # batched = quantization kernel + contraction


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
def cpu_reference_run(steps: int, warmup: int, nl: int = 2):
    """Times the reference's own CPU kernel (bitnet_gemm_i2_i8 compiled from its sources, behind
    oracle/_ref) on a bounded sample of the sweep; falls back to the C port of the oracle."""
    import numpy as np

    from oracle import bitlinear_oracle as O
    from oracle.clib import load_oracle, load_reference

    ref = load_reference()
    kind = "reference" if ref is not None else "port"
    port = load_oracle()
    cores = ref.num_threads() if ref is not None else port.num_threads()
    rng = np.random.default_rng(0)
    # nl layers per shape in the sample, rotated so the weights do not stay in the cores' L1/L2
    work = []
    for (n, k) in SHAPES:
        mats = []
        for _ in range(nl):
            t = rng.integers(-1, 2, size=(n, k)).astype(np.int8)
            mats.append(O.pack_i2s(t) if ref is not None else port.pack_wf16(t))
        for m in BATCHES:
            q = rng.integers(-127, 128, size=(m, k)).astype(np.int8)
            work.append((n, k, m, mats, q))

    def one_step():
        for (n, k, m, mats, q) in work:
            for p in mats:
                if ref is not None:
                    ref.gemm(p, q, 0.02)
                else:
                    port.gemm_wf16(q, p)

    bytes_step = sum(algorithmic_bytes(m, n, k) * nl for (n, k, m, _, _) in work)
    for _ in range(warmup):
        one_step()
    t0 = time.perf_counter()
    for _ in range(steps):
        one_step()
    dt = (time.perf_counter() - t0) / steps
    sample = (f"{nl} layers per shape x 3 shapes x M in {BATCHES}, int8 activations already quantized, "
              f"{steps} steps of {dt * 1e3:.1f} ms; kernel: " +
              ("bitnet_gemm_i2_i8 (AVX-%s build of the reference's bitnet_gemv.cpp, OpenMP)" % ref.flavour.replace("avx", "")
               if ref is not None else "scalar C port of the oracle (OpenMP)"))
    return dict(value=bytes_step / dt / 1e9, unit="GB/s", cores=cores, kind=kind, sample=sample), steps, warmup, dt


# ------------------------------------------------------------------ prefill GEMM (secondary figures of the same line)
PREFILL_M = [512, 2048, 8192]


def prefill_section(wf, torch, device, peaks, shapes=None, ms=None):
    """int8 x ternary GEMM on tcgen05 at the sweep's shapes: TOPS = 2*M*N*K / time, for the whole operator
    (activation quantization + contraction) with bf16 activations resident in HBM."""
    out = []
    gd = torch.Generator(device=device).manual_seed(4242)
    for (n, k) in (shapes or [(2560, 2560), (6912, 2560), (2560, 6912)]):
        codes, scale = wf.pack_ternary(torch.randn(n, k, generator=gd, device=device) * 0.02)
        for m in (ms or PREFILL_M):
            x = torch.randn(m, k, generator=gd, device=device).to(torch.bfloat16)
            y = torch.empty(m, n, dtype=torch.bfloat16, device=device)
            graph = capture(torch, lambda: wf.bitlinear(x, codes, scale, out=y, path="prefill"))
            for _ in range(3):
                graph.replay()
            torch.cuda.synchronize()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            reps = 10
            a.record()
            for _ in range(reps):
                graph.replay()
            b.record()
            torch.cuda.synchronize()
            us = a.elapsed_time(b) * 1e3 / reps
            tops = 2.0 * m * n * k / us / 1e6
            out.append({"N": n, "K": k, "M": m, "us": round(us, 2), "TOPS": round(tops, 1),
                        "frac_of_2x_measured_bf16": round(tops / (2 * peaks["bf16_tflops"]), 4),
                        "frac_of_nominal_int8_4500": round(tops / 4500.0, 4)})
    return out


# ------------------------------------------------------------------ decoder tokens/s (secondary figures)
def decoder_section(wf, torch, device, world, full: bool):
    """Greedy decode tokens/s of random-init ternary decoders on the BitLinear kernels (CUDA-graphed step):
    Llama-3-8B shape at a 2048-token context for batch 1 and 32 (256 with --decoder-full), tensor-parallel over
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
        model = TernaryDecoder(LLAMA3_8B, batch, 2048, device, seed=7)
        for L in model.layers:  # a context of 2048 random tokens' keys and values
            L["kc"].normal_()
            L["vc"].normal_()
        model.pos.fill_(2047)
        model.capture(masked=False)
        ms = timed(model, 16)
        by = model.weight_bytes_per_step()
        out.append({"model": "llama3-8b-shape", "tp": world, "batch": batch, "context": 2048, "ms_per_step": round(ms, 3),
                    "tok_s": round(batch / ms * 1e3, 1), "GB_per_step_per_rank": round(by / 1e9, 3),
                    "GBps_per_rank": round(by / ms / 1e6, 1)})
        del model
        torch.cuda.empty_cache()
    if world == 1:
        model = TernaryDecoder(SMOLLM2_135M, 32, 640, device, seed=8)
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
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--layers-scale", type=float, default=1.0, help="scale the layer stacks (profiling on a small case)")
    ap.add_argument("--no-pdl", action="store_true")
    ap.add_argument("--prefill-only", action="store_true", help="run only the prefill GEMM section (profiling)")
    ap.add_argument("--no-decoder", action="store_true", help="skip the decoder tokens/s section")
    ap.add_argument("--decoder-only", action="store_true", help="run only the decoder tokens/s section (profiling)")
    ap.add_argument("--decoder-full", action="store_true", help="also batch 256 of the 8B shape")
    ap.add_argument("--only-m", type=int, default=0, help="restrict the sweep to one token batch (profiling)")
    ap.add_argument("--only-shape", type=int, default=-1, help="restrict the sweep to one shape index (profiling)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    warmup = max(args.warmup, 3)
    config = {"workload": "decode_gemv_sweep", "shapes_NxK": ["%dx%d" % s for s in SHAPES], "batches_M": BATCHES,
              "layers_per_shape": [LAYERS[s] for s in SHAPES], "activations": "bf16 N(0,1) + 0.1% outliers at +-20",
              "weights": "N(0,0.02) absmean-ternarized, 2 bits/weight", "l2": "inputs larger than L2 (distinct weights per launch)"}

    if args.impl == "reference":
        if rank != 0:
            return
        cb, steps, wu, dt = cpu_reference_run(args.steps, warmup)
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
        res = decoder_section(wf, torch, device, world, args.decoder_full)
        if rank == 0:
            print(json.dumps({"decode_tok_s": res}))
        return
    if args.prefill_only:
        peaks, _ = measured_peaks()
        res = prefill_section(wf, torch, device, peaks, [SHAPES[args.only_shape]] if args.only_shape >= 0 else None,
                              [args.only_m] if args.only_m else None)
        print(json.dumps({"prefill_gemm": res}))
        return
    if args.only_m:
        BATCHES[:] = [args.only_m]
    if args.only_shape >= 0:
        SHAPES[:] = [SHAPES[args.only_shape]]
    note(rank, "building workload")
    groups = build_workload(wf, torch, device, rank, world, args.layers_scale)
    note(rank, "capturing step graph")
    pdl = not args.no_pdl
    try:
        graph = capture(torch, lambda: run_step(wf, groups, pdl))
    except RuntimeError as e:  # programmatic dependent launch not capturable here: plain edges
        if not pdl:
            raise
        print(f"[bench] capture with programmatic dependent launch failed ({e}); retrying without", file=sys.stderr)
        pdl = False
        torch.cuda.synchronize()
        graph = capture(torch, lambda: run_step(wf, groups, pdl))
    launches = sum(2 if g["batched"] else 1 for g in groups)
    total_bytes = step_bytes(groups)

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    note(rank, "device-resident timing")
    # ---- device-resident timing
    for _ in range(warmup):
        graph.replay()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
        time.sleep(0.3)
    barrier()  # after the sampler is up: no rank may enter the timed region ahead of the others
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ev0.record()
    for _ in range(args.steps):
        graph.replay()
    ev1.record()
    barrier()
    ms = ev0.elapsed_time(ev1) / args.steps
    clocks = sampler.finish() if rank == 0 else None

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
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    e2e_fork()
    for _ in range(args.steps):
        e2e_step()
    e2e_join()
    e1.record()
    barrier()
    ms_e2e = e0.elapsed_time(e1) / args.steps

    if dist is not None:
        t = torch.tensor([ms, ms_e2e], device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms, ms_e2e = t.tolist()
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
        gr = capture(torch, lambda: run_step(wf, gs, pdl))
        for _ in range(3):
            gr.replay()
        barrier()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(args.steps):
            gr.replay()
        b.record()
        barrier()
        t = a.elapsed_time(b) / args.steps
        if dist is not None:
            tt = torch.tensor([t], device=device)
            dist.all_reduce(tt, op=dist.ReduceOp.MAX)
            t = tt.item()
        return t

    note(rank, "timing kernel families")
    ms_dec, ms_gemm = time_groups(dec_groups), time_groups(gemm_groups)
    note(rank, "breakdown")
    gemm_ops = sum(2.0 * g["m"] * g["n"] * g["k"] * len(g["layers"]) for g in gemm_groups)
    n_gemm_groups = len(gemm_groups)
    dec_launches = max(1, len(dec_groups))
    per_launch_bytes = step_bytes(dec_groups) / dec_launches / world if dec_groups else 0.0  # what one rank's kernel moves
    per_launch_us = (ms_dec or 0.0) * 1e3 / dec_launches
    achieved = per_launch_bytes / (per_launch_us * 1e-6) / 1e9 if dec_groups else 0.0
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
        a.record()
        reps = 10
        for _ in range(reps):
            gr.replay()
        b.record()
        torch.cuda.synchronize()
        us = a.elapsed_time(b) * 1e3 / reps / len(g["layers"])
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
            decoder = decoder_section(wf, torch, device, world, args.decoder_full)
        except Exception as e:  # the main line must survive a failure of this secondary section
            decoder = [{"error": repr(e)[:300]}]
    note(rank, "done with collective phases")
    if rank != 0:
        # stay in step with rank 0 (it still runs single-GPU sections): tear the group down together
        finish(dist, torch, rank)
        return
    line = {"metric": METRIC, "value": value, "unit": "GB/s", "n_gpus": world, "steps": args.steps, "warmup": warmup,
            "ms_per_step": ms, "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "u8xs8->s32",
            "data": "synthetic", "config": dict(config, pdl=pdl, graph=True, parallelism=f"tp{world}" if world > 1 else "single"),
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                         "frac": achieved / peaks["hbm_gbs"], "traffic": per_launch_bytes * NCU_TRAFFIC_RATIO,
                         "traffic_source": "ncu capture of the M=1 2560x2560 group (203.5 MB DRAM for 197.8 MB algorithmic), scaled",
                         "peak_kind": peak_kind + " copy bandwidth",
                         "kernel": "decode_stream_kernel", "launches": f"the {dec_launches} grouped launches with M < {GEMM_MIN_M}",
                         "bytes_per_launch": per_launch_bytes, "us_per_launch": per_launch_us},
            "e2e": {"value": full_bytes / (ms_e2e * 1e-3) / 1e9, "unit": "GB/s", "h2d_bytes_per_step": h2d,
                    "d2h_bytes_per_step": d2h, "ms_per_step": ms_e2e},
            "gpu_launches": launches * args.steps, "clocks": clocks, "breakdown": breakdown}
    if n_gemm_groups and ms_gemm:
        tops = gemm_ops / (ms_gemm * 1e-3) / 1e12
        line["roofline_gemm"] = {"bound": "tensor", "kernel": "prefill_kernel (batched over each layer stack)",
                                 "launches": f"the {n_gemm_groups} stacks with M >= {GEMM_MIN_M}", "achieved": tops,
                                 "unit": "TOPS", "peak": 2 * peaks["bf16_tflops"],
                                 "peak_kind": "2 x measured bf16 burst (int8 dense proxy; nominal 4500)",
                                 "frac": tops / (2 * peaks["bf16_tflops"]), "ms": ms_gemm,
                                 "note": "useful ops 2*M*N*K; the 128-token MMA tile is partly padding at M = 16 and 64"}
    if decoder is not None:
        line["decode_tok_s"] = decoder
    if not args.only_m and args.only_shape < 0:
        note(rank, "prefill GEMM section")
        line["prefill_gemm"] = prefill_section(wf, torch, device, peaks)
        note(rank, "prefill GEMM section done")
    if not args.no_cpu_baseline and world == 1:
        cb, _, _, _ = cpu_reference_run(3, 1)
        line["cpu_baseline"] = cb
    print(json.dumps(line), flush=True)
    if dist is not None:
        finish(dist, torch, rank)


if __name__ == "__main__":
    main()
