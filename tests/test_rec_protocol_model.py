"""Model of the barrier protocol of the recurrence kernel (csrc/chunkwise_sm100.cu, rec_sm100), run on the CPU.

Six roles hand work around two rings whose barriers run on over the whole sequence (thousands of phases), every wait
seeing only the phase PARITY: the TMA producer (ring of four half-chunk stages), the gating warps, the MMA thread (two
accumulator buffers), the state warps, the store warp (two staging buffers) and the n warp (two buffers of partial
sums).  The order of waits, arrivals, copy issues and MMA commits of each role is restated here and run under random
interleavings - copies land in any order, commits fire in order - with every wait checked against the true phase
count (a waiter two phases away from its barrier, early or late, is a hang or a corruption), every barrier against
over-arrival, the run against deadlock, and the eight-entry ring of chunk decays against being overwritten before
its readers are done.  A model, kept next to the kernel by hand."""

import random

import pytest


class Bar:
    def __init__(self, name, count):
        self.name, self.count, self.pending, self.phase = name, count, count, 0

    def arrive(self):
        self.pending -= 1
        assert self.pending >= 0, f"over-arrival on {self.name}"
        if self.pending == 0:
            self.phase += 1
            self.pending = self.count

    def test(self, want):
        passes = (self.phase & 1) != (want & 1)      # what the hardware sees
        truth = self.phase > want
        if passes and not truth:
            raise AssertionError(f"ALIAS early pass on {self.name}: want {want} at {self.phase}")
        if truth and not passes:
            raise AssertionError(f"ALIAS late wait on {self.name}: want {want} at {self.phase}")
        return passes


def run(NC, do_n, store_states, seed, stages=4):
    rnd = random.Random(seed)
    NH2 = 2 * NC
    B = {}
    for s in range(stages):
        B[f"full{s}"], B[f"empty{s}"], B[f"scaled{s}"] = Bar(f"full{s}", 1), Bar(f"empty{s}", 1), Bar(f"scaled{s}", 8)
    for s in range(2):
        B[f"acc_full{s}"], B[f"acc_free{s}"] = Bar(f"acc_full{s}", 1), Bar(f"acc_free{s}", 8)
        B[f"nsum{s}"], B[f"nread{s}"] = Bar(f"nsum{s}", 8), Bar(f"nread{s}", 1)
        B[f"out_full{s}"], B[f"out_free{s}"] = Bar(f"out_full{s}", 8), Bar(f"out_free{s}", 1)
    loads, commits = [], []          # copies in flight (land in any order), MMA commits (fire in order)
    decay_written = [-1] * 8         # chunk whose decay sits in each slot of the ring of eight
    state_done = [-1] * 8            # last chunk each state warp has folded (it reads the chunk's decay while folding)
    n_done = [-1 if do_n else 10 ** 9]

    def producer():
        for h in range(NH2):
            st, s = h % stages, h >> 1
            if h % 2 == 0:
                if decay_written[s & 7] >= 0:   # about to overwrite the decay of chunk s - 8
                    assert min(state_done + n_done) >= decay_written[s & 7], "decay ring overwritten too early"
                decay_written[s & 7] = s
            yield ("wait", f"empty{st}", h // stages - 1)
            loads.append(st)
            yield ("step",)

    def mma():
        for h in range(NH2):
            st, s = h % stages, h >> 1
            buf = s & 1
            yield ("wait", f"scaled{st}", h // stages)
            if h % 2 == 0:
                yield ("wait", f"acc_free{buf}", (s >> 1) - 1)
            commits.append(f"empty{st}")
            if h % 2 == 1:
                commits.append(f"acc_full{buf}")

    def gating():
        for h in range(NH2):
            st, s = h % stages, h >> 1
            nb = s & 1
            yield ("wait", f"full{st}", h // stages)
            if do_n and h % 2 == 1 and s >= 2:
                yield ("wait", f"nread{nb}", (s >> 1) - 1)
            B[f"scaled{st}"].arrive()
            if do_n and h % 2 == 1:
                B[f"nsum{nb}"].arrive()

    def store_warp():
        for n in range(NC + 1):
            ob = n & 1
            yield ("wait", f"out_full{ob}", n >> 1)
            if n >= 1:
                B[f"out_free{ob ^ 1}"].arrive()

    def n_warp():
        for s in range(NC):
            nb = s & 1
            yield ("wait", f"nsum{nb}", s >> 1)
            B[f"nread{nb}"].arrive()
            n_done[0] = s

    def state_warp(w):
        n_out = 0

        def store_c():
            nonlocal n_out
            if store_states:
                ob = n_out & 1
                if n_out >= 2:
                    yield ("wait", f"out_free{ob}", (n_out >> 1) - 1)
                B[f"out_full{ob}"].arrive()
            n_out += 1
        yield from store_c()
        for s in range(NC):
            buf = s & 1
            yield ("wait", f"acc_full{buf}", s >> 1)
            B[f"acc_free{buf}"].arrive()
            state_done[w] = s
            yield from store_c()

    agents = {"prod": producer(), "mma": mma()}
    for w in range(8):
        agents[f"gate{w}"] = gating()
        agents[f"state{w}"] = state_warp(w)
    if store_states:
        agents["store"] = store_warp()
    if do_n:
        agents["n"] = n_warp()
    blocked, alive = {}, set(agents)
    while alive:
        choices = [("agent", a) for a in alive]
        if loads:
            choices.append(("load", None))
        if commits:
            choices.append(("commit", None))
        rnd.shuffle(choices)
        progressed = False
        for kind, a in choices:
            if kind == "load":
                B[f"full{loads.pop(rnd.randrange(len(loads)))}"].arrive()
                progressed = True
                break
            if kind == "commit":
                B[commits.pop(0)].arrive()
                progressed = True
                break
            if a in blocked:
                _, bn, ph = blocked[a]
                if not B[bn].test(ph):
                    continue
                del blocked[a]
            try:
                op = next(agents[a])
            except StopIteration:
                alive.discard(a)
                progressed = True
                break
            if op[0] == "wait" and not B[op[1]].test(op[2]):
                blocked[a] = op
            progressed = True
            break
        if not progressed:
            raise AssertionError(f"DEADLOCK: {blocked}")


@pytest.mark.parametrize("NC", [1, 2, 3, 5, 8, 17, 40])
@pytest.mark.parametrize("do_n,store_states", [(True, True), (False, True), (False, False), (True, False)])
def test_recurrence_protocol_has_no_aliasing_deadlock_or_over_arrival(NC, do_n, store_states):
    for seed in range(25):
        run(NC, do_n, store_states, seed)
