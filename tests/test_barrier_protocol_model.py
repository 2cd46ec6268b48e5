"""Model of the barrier protocol of the intra-chunk kernels (csrc/chunkwise_sm100.cu, par_body), run on the CPU.

The kernel's three roles - the TMA producer thread, the MMA thread and the eight element-wise warps - hand work to each
other through mbarriers, and an mbarrier wait sees only the PARITY of the phase it waits for.  A wait is therefore only
safe if the waiter can never be two phases away from the barrier, in either direction: two ahead, and it passes on the
previous occupant's completion (reading a stage the copy engine is still filling); two behind, and it sleeps through
the completion it wants.  This file restates the order of waits, arrivals, load issues and MMA commits of each role
(one chunk per CTA, 1 to 8 output tiles, 2 to 8 operand slices, with and without the extra E tile) and runs them under
random interleavings - asynchronous copies land in any order, MMA commits fire in order - checking every wait against
the true phase count, every barrier against over-arrival, and the whole run against deadlock.

It is a model, kept next to the kernel by hand: change the order of barrier operations in par_body and this file has
to follow.  Its second test documents why a CTA does not walk several chunks with the ring running on: the MMA thread
would then poll a stage's `full` barrier while the previous chunk's E tile is still in flight on it."""

import random

import pytest

class Bar:
    def __init__(self, name, count):
        self.name, self.count, self.pending, self.phase = name, count, count, 0
    def arrive(self):
        self.pending -= 1
        assert self.pending >= 0, f"over-arrival on {self.name}"
        if self.pending == 0:
            self.phase += 1; self.pending = self.count
    def test(self, want_phase):
        # hardware sees only parity: passes when current phase parity != parity of want_phase
        passes = (self.phase & 1) != (want_phase & 1)
        truth = self.phase > want_phase
        if passes != truth:
            if passes: raise AssertionError(f"ALIAS early pass on {self.name}: want {want_phase} at {self.phase}")
            # blocked although complete (barrier two phases ahead): would hang
            if self.phase >= want_phase + 2: raise AssertionError(f"ALIAS hang on {self.name}: want {want_phase} at {self.phase}")
        return passes

def run(mode, ND, nsub, njobs, seed, NST=3):
    rnd = random.Random(seed)
    HAS_E = mode in ("DQ", "DK")
    n0 = 2 * ND + 1 + (1 if HAS_E else 0); n1 = ND + 1 + (1 if HAS_E else 0)
    n_loads = n0 + (nsub - 1) * n1
    B = {}
    for s in range(NST):
        B[f"full{s}"] = Bar(f"full{s}", 1); B[f"empty{s}"] = Bar(f"empty{s}", 1)
    for n, c in (("sfull",1),("afull",1),("hfull",1),("gated",8),("accfree",8),("done",8),("dot",8),("out",8)):
        B[n] = Bar(n, c)
    for qd in range(4): B[f"pair{qd}"] = Bar(f"pair{qd}", 2)
    pending_async = []   # async completions: ('load', st) any order ; commits in order
    commit_queue = []    # list of barrier names, fire in order
    def kind_of(sub, l):
        if sub == 0 and l < ND: return "SCORE"
        ls = l - (ND if sub == 0 else 0)
        if ls < ND: return "STATE"
        return "X" if ls == ND else "E"
    # generators for each role; yield ('wait', barname, phase) blocks until passes; other ops executed inline
    def producer():
        issued = 0; rm = [0]*NST; st = 0; hist = []
        for job in range(njobs):
            sub = 0; l = 0
            for ld in range(n_loads):
                kind = kind_of(sub, l)
                if issued >= NST:
                    pk, ps = hist[-3]
                    if pk in ("SCORE", "STATE") or (pk == "X" and HAS_E):
                        yield ("wait", f"empty{st}", rm[st] - 1)
                    else:
                        yield ("wait", "done", ps)
                pending_async.append(("load", st))
                if kind in ("SCORE", "STATE") or (kind == "X" and HAS_E): rm[st] += 1
                issued += 1
                hist.append((kind, job * nsub + sub))
                st = (st + 1) % NST
                l += 1
                if l == (n0 if sub == 0 else n1): l = 0; sub += 1
                yield ("step",)
    def mma():
        for job in range(njobs):
            lb = job * n_loads; gt0 = job * nsub
            for ld in range(ND):
                gl = lb + ld; st = gl % NST
                yield ("wait", f"full{st}", gl // NST)
                commit_queue.append(f"empty{st}")
            commit_queue.append("sfull")
            for sub in range(nsub):
                gt = gt0 + sub
                lbase = lb + (ND if sub == 0 else n0 + (sub - 1) * n1)
                if gt > 0: yield ("wait", "accfree", gt - 1)
                for it in range(ND):
                    ld = lbase + it; st = ld % NST
                    yield ("wait", f"full{st}", ld // NST)
                    commit_queue.append(f"empty{st}")
                commit_queue.append("afull")
                ldx = lbase + ND; stx = ldx % NST
                yield ("wait", f"full{stx}", ldx // NST)
                yield ("wait", "gated", gt)
                if HAS_E: commit_queue.append(f"empty{stx}")
                commit_queue.append("hfull")
    def ew(quarter, half):
        for job in range(njobs):
            lb = job * n_loads; gt0 = job * nsub
            yield ("barsync",)
            yield ("wait", "sfull", job)
            B[f"pair{quarter}"].arrive()
            yield ("wait", f"pair{quarter}", job)
            for sub in range(nsub):
                gt = gt0 + sub
                yield ("wait", "afull", gt)
                B["gated"].arrive()
                yield ("wait", "hfull", gt)
                ldx = lb + (2 * ND if sub == 0 else n0 + (sub - 1) * n1 + ND)
                if HAS_E:
                    lde = ldx + 1; ste = lde % NST
                    yield ("wait", f"full{ste}", lde // NST)
                # the shipped kernel (one chunk per CTA) hands the accumulator and the staging stage back only when
                # another tile follows; with the ring running on across chunks every tile has to
                if njobs > 1 or sub + 1 < nsub: B["accfree"].arrive()
                B["out"].arrive()
                yield ("wait", "out", gt)
                if HAS_E:
                    B["dot"].arrive()
                    if half == 0: yield ("wait", "dot", gt)
                if njobs > 1 or sub + 1 < nsub: B["done"].arrive()
    agents = {"prod": producer(), "mma": mma()}
    for qd in range(4):
        for h in range(2): agents[f"ew{qd}{h}"] = ew(qd, h)
    blocked = {}
    barsync_wait = set()
    alive = set(agents)
    steps = 0
    while alive:
        steps += 1
        choices = []
        for a in alive:
            if a in barsync_wait: continue
            choices.append(("agent", a))
        if pending_async: choices.append(("async_load", None))
        if commit_queue: choices.append(("commit", None))
        # try a random choice; if agent blocked, it stays blocked
        rnd.shuffle(choices)
        progressed = False
        for ch in choices:
            if ch[0] == "async_load":
                i = rnd.randrange(len(pending_async)); _, st = pending_async.pop(i)
                B[f"full{st}"].arrive(); progressed = True; break
            if ch[0] == "commit":
                B[commit_queue.pop(0)].arrive(); progressed = True; break
            a = ch[1]
            if a in blocked:
                _, bn, ph = blocked[a]
                try:
                    okk = B[bn].test(ph)
                except AssertionError as e:
                    raise AssertionError(f"{a}: {e}")
                if okk: del blocked[a]
                else: continue
            try:
                op = next(agents[a])
            except StopIteration:
                alive.discard(a); progressed = True; break
            if op[0] == "wait":
                try:
                    okk = B[op[1]].test(op[2])
                except AssertionError as e:
                    raise AssertionError(f"{a}: {e}")
                if not okk: blocked[a] = op
                progressed = True; break
            if op[0] == "barsync":
                barsync_wait.add(a)
                if len(barsync_wait) == 8: barsync_wait.clear()
                progressed = True; break
            progressed = True; break
        if not progressed:
            raise AssertionError(f"DEADLOCK: blocked={blocked} barsync={barsync_wait} phases={{k:v.phase for k,v in B.items()}}".replace("{{","{").replace("}}","}") + str({k:v.phase for k,v in B.items()}))
    return steps



MODES = ("H", "DV", "DK", "DQ")   # H and DV: no E tile (the output is staged in the X tile's stage)


@pytest.mark.parametrize("mode", MODES)
@pytest.mark.parametrize("ND", [2, 4, 8])
@pytest.mark.parametrize("nsub", [1, 2, 3, 4, 8])
def test_one_chunk_per_cta_protocol_has_no_aliasing_deadlock_or_over_arrival(mode, ND, nsub):
    for seed in range(40):
        run(mode, ND, nsub, 1, seed)


def test_ring_running_on_across_chunks_would_alias():
    """Several chunks per CTA with the ring and barriers running on (tried and taken out): some interleaving lets a
    waiter meet a barrier two phases away."""
    for seed in range(4000):
        try:
            run("DQ", 8, 3, 8, seed)
        except AssertionError as e:
            assert "ALIAS" in str(e)
            return
    raise AssertionError("no interleaving out of 4000 showed the hazard")
