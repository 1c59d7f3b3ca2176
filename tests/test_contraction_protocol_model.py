"""A model of the barrier protocol of the tensor-core contraction (csrc/wf_prefill.cu, single form), run under random
interleavings: the two TMA loaders, eight expansion warps, the issuing threads, their asynchronous MMA completions and the
epilogue warps, with the kernel's barrier counts and parity arithmetic (mbarrier waits succeed when the barrier's phase
parity differs from the one waited for, so a waiter that falls two phases behind would be caught as a hang).  Checked
for every form the kernel has (issuing threads, ring slots, accumulator buffers) and for stage counts below, at and above
the number of issuing threads: no wait is passed early (a stage is issued only on a slot that holds its expanded weights
and its token tile), no slot is overwritten while its MMAs are in flight, a tile's accumulators are read only when all
its MMAs are complete and overwritten only after they were read, and every role runs to its end.
This is a model of the protocol, not of the hardware: it guards the bookkeeping (counts, parities, ring arithmetic)
against edits."""
import random

import pytest


class Bar:
    def __init__(self, count, name):
        self.count, self.pending, self.phase, self.name = count, count, 0, name
    def arrive(self):
        self.pending -= 1
        assert self.pending >= 0, f"{self.name}: more arrivals than the count in phase {self.phase}"
        if self.pending == 0:
            self.phase += 1
            self.pending = self.count
    def test(self, parity):
        return (self.phase & 1) != parity

def run(NI, XS, BUFS, stages, tiles, EPI_WARPS, PS=6, seed=0, steps_limit=2_000_000):
    rnd = random.Random(seed)
    p_full = [Bar(1, f"p_full{i}") for i in range(PS)]
    p_empty = [Bar(8, f"p_empty{i}") for i in range(PS)]
    a_full = [Bar(9, f"a_full{i}") for i in range(XS)]
    st_free = [Bar(1, f"st_free{i}") for i in range(XS)]
    acc_full = [Bar(NI, f"acc_full{i}") for i in range(2)]
    acc_empty = [Bar(EPI_WARPS, f"acc_empty{i}") for i in range(2)]
    # ground truth state for hazard checks
    slot_stage = [-1] * XS          # stage whose expanded weights the slot holds (complete when writers == 8)
    slot_writers = [0] * XS
    slot_x = [-1] * XS              # stage whose token tile the slot holds
    mma_done = set()                # stages whose MMAs have completed
    mma_issued = set()
    tile_loaded = set()             # tiles whose accumulators the epilogue has read (per epilogue warp count)
    tile_loads = {}
    fifo = [[] for _ in range(NI)]  # per issuing thread: queue of ('mma', stage) / ('commit', bar)
    errors = []

    def W(bar, parity):  # a wait: generator yields until passes
        while not bar.test(parity):
            yield

    def loaderP():
        for sit in range(tiles * stages):
            s = sit % PS
            if sit >= PS:
                yield from W(p_empty[s], ((sit // PS) - 1) & 1)
            p_full[s].arrive()
            yield
    def loaderX():
        for sit in range(tiles * stages):
            s = sit % XS
            if sit >= XS:
                yield from W(st_free[s], ((sit // XS) - 1) & 1)
            if sit >= XS and (sit - XS) not in mma_done:
                errors.append(f"token tile of stage {sit} overwrites slot {s} while stage {sit - XS} is still in use")
            slot_x[s] = sit
            a_full[s].arrive()
            yield
    def expander(w):
        for sit in range(tiles * stages):
            ps, s = sit % PS, sit % XS
            yield from W(p_full[ps], (sit // PS) & 1)
            yield
            if sit >= XS:
                yield from W(st_free[s], ((sit // XS) - 1) & 1)
            if sit >= XS and (sit - XS) not in mma_done:
                errors.append(f"expansion of stage {sit} overwrites slot {s} while stage {sit - XS} is still in use")
            if slot_stage[s] != sit:
                slot_stage[s], slot_writers[s] = sit, 0
            slot_writers[s] += 1
            yield
            p_empty[ps].arrive()
            a_full[s].arrive()
            yield
    def issuer(i):
        nt, sit0 = 0, 0
        for t in range(tiles):
            a = nt % BUFS
            r0 = sit0 % NI
            g0 = i - r0 if i >= r0 else i - r0 + NI
            if nt >= BUFS:
                yield from W(acc_empty[a], ((nt // BUFS) - 1) & 1)
                if tile_loads.get(nt - BUFS, 0) != EPI_WARPS:
                    errors.append(f"issuer {i} starts tile {nt} before tile {nt - BUFS} has been read")
            if g0 >= stages:
                acc_full[a].arrive()
            else:
                for g in range(g0, stages, NI):
                    sit = sit0 + g
                    s = sit % XS
                    yield from W(a_full[s], (sit // XS) & 1)
                    if slot_stage[s] != sit or slot_writers[s] != 8 or slot_x[s] != sit:
                        errors.append(f"issuer {i}: stage {sit} issued on slot {s} holding stage {slot_stage[s]} ({slot_writers[s]} writers), tokens of {slot_x[s]}")
                    mma_issued.add(sit)
                    fifo[i].append(("mma", sit))
                    fifo[i].append(("commit", st_free[s]))
                    yield
                fifo[i].append(("commit", acc_full[a]))
            nt += 1
            sit0 += stages
            yield
    def pipe(i):  # completes this thread's operations in order, at random times
        while True:
            if fifo[i]:
                kind, v = fifo[i].pop(0)
                if kind == "mma":
                    mma_done.add(v)
                else:
                    v.arrive()
            yield
    def epilogue(w):
        for nt in range(tiles):
            a = nt % BUFS
            yield from W(acc_full[a], (nt // BUFS) & 1)
            first, last = nt * stages, nt * stages + stages - 1
            if not all(sg in mma_done for sg in range(first, last + 1)):
                errors.append(f"epilogue reads tile {nt} before its MMAs are complete")
            tile_loads[nt] = tile_loads.get(nt, 0) + 1
            yield
            acc_empty[a].arrive()
            for _ in range(rnd.randint(0, 6)):
                yield  # rescale and store

    roles = {"P": loaderP(), "X": loaderX()}
    for w in range(8):
        roles[f"E{w}"] = expander(w)
    for i in range(NI):
        roles[f"I{i}"] = issuer(i)
    for w in range(EPI_WARPS):
        roles[f"O{w}"] = epilogue(w)
    daemons = {f"T{i}": pipe(i) for i in range(NI)}
    live = dict(roles)
    steps = 0
    weights = {k: rnd.choice([1, 1, 2, 5]) for k in list(live) + list(daemons)}
    idle = 0
    while live and steps < steps_limit and not errors:
        names = list(live) + list(daemons)
        k = rnd.choices(names, [weights[n] for n in names])[0]
        steps += 1
        if k in daemons:
            next(daemons[k])
            continue
        try:
            next(live[k])
        except StopIteration:
            del live[k]
        except AssertionError as e:
            errors.append(str(e))
    if live and not errors:
        errors.append(f"no progress: still running {sorted(live)}")
    return errors



# (issuing threads, ring slots, accumulator buffers, epilogue warps) of the forms for 16 / 32-64 / 128 and more tokens
FORMS = {"16 tokens": (3, 3, 2, 4), "32 and 64 tokens": (2, 2, 2, 8), "128 tokens": (1, 2, 2, 8)}


@pytest.mark.parametrize("form", sorted(FORMS))
@pytest.mark.parametrize("stages", [1, 2, 3, 5, 7, 14])
def test_protocol_model(form, stages):
    ni, xs, bufs, epi = FORMS[form]
    for seed in range(3):
        errs = run(ni, xs, bufs, stages, tiles=7, EPI_WARPS=epi, seed=seed)
        assert not errs, (form, stages, seed, errs[:2])
