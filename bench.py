#!/usr/bin/env python
"""Benchmark of the mLSTM hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl b200|reference]

One step = one chunkwise mLSTMexp forward+backward over one synthetic 65,536-token batch
(B=8, S=8192, NH=16, DHQK=DHHV=256, chunk 128, bf16; seeded q,k,v,i ~ N(0,1), f = 3 + N(0,1),
dH ~ N(0,1)), per-chunk states kept for the backward (recompute_states_in_bw=False; the recompute setting is
timed next to it).  With N > 1 (torchrun, one rank per GPU) every rank processes its own batch of the same size:
batch x heads are independent units, there is no data-path collective (weak scaling).  The same run also
measures, under `extra`, the FIXED batch sharded over the N ranks (strong scaling), decode sharded over batch
and the sequence-parallel prefill of one long sequence over the N ranks.

Prints ONE JSON line.  `value` is TFLOP/s of algorithmic FLOPs with inputs resident in HBM;
`e2e` is the same metric through the public API with host (pinned) buffers, host<->device copies
inside the timed region.  `--impl reference` times the reference's own native PyTorch chunkwise path
(mlstm_chunkwise__native_custbw, fp32, CPU, all host threads) on a bounded sample of the same workload; when the
reference package cannot be imported it falls back to the numpy restatement of that algorithm (the oracle).
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

# torchrun exports OMP_NUM_THREADS=1 for every rank; the CPU baseline legs must use all host cores, so undo that
# before numpy / torch load their BLAS and OpenMP runtimes.
if os.environ.get("OMP_NUM_THREADS") == "1":
    os.environ["OMP_NUM_THREADS"] = str(os.cpu_count() or 1)

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))
REF_DIR = os.path.join(ROOT, "baseline", "_ref")

WORKLOAD = dict(name="c2_chunkwise_fwbw_mLSTMexp_B8_S8192_NH16_DHQK256_DHHV256_L128_bf16",
                B=8, S=8192, NH=16, DHQK=256, DHHV=256, L=128)
# bounded CPU sample of the same workload: same S, head dims and chunk size, fewer (batch, head) units
CPU_SAMPLE = dict(B=1, NH=16)
METRIC = "chunkwise_fwbw_tflops_64k_tokens"


# measured with ncu (dram__bytes_read.sum + dram__bytes_write.sum) at NH=16, 256/256, chunk 128, bf16 on a quarter
# batch, divided by its 2048 chunks; the ncu summaries are kept under profiles/
NCU_DRAM_BYTES_PER_CHUNK = {"recurrent_fw": 246736, "parallel_fw": 389655, "recurrent_bw": 244795, "parallel_bw": 717398}


def fw_flops(B, NH, S, DHQK, DHHV, L):
    return B * NH * S * (4 * DHQK * DHHV + L * (DHQK + DHHV))


def bw_flops(B, NH, S, DHQK, DHHV, L):
    return B * NH * S * (8 * DHQK * DHHV + L * (3 * DHQK + 2 * DHHV))


def phase_flops(B, NH, S, DHQK, DHHV, L):
    t = B * NH * S
    return {
        "recurrent_fw": t * 2 * DHQK * DHHV,
        "parallel_fw": t * (2 * DHQK * DHHV + L * (DHQK + DHHV)),
        "recurrent_bw": t * 2 * DHQK * DHHV,
        "parallel_bw": t * (6 * DHQK * DHHV + L * (3 * DHQK + 2 * DHHV)),
    }


def step_bytes(B, NH, DHQK, DHHV):
    return B * NH * (2 * DHQK * DHHV * 4 + 2 * DHQK * 4 + 8 + (2 * DHQK + 2 * DHHV) * 2 + 4)


def measured_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return dict(tflops=d["bf16_tflops"], tflops_sustained=d.get("bf16_tflops_sustained"), hbm=d["hbm_gbs"],
                    source="measured")
    return dict(tflops=1590.0, tflops_sustained=1400.0, hbm=6650.0, source="fallback")


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu = gpu_index
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.gpu}", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is None:
            return dict(sm_mhz=None, sm_max_mhz=None, reasons=["nvidia-smi unavailable"])
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in self.lines:
            parts = [p.strip() for p in ln.split(",")]
            if len(parts) < 9:
                continue
            try:
                sm.append(float(parts[1])); mx.append(float(parts[2]))
            except ValueError:
                continue
            for nm, val in zip(names, parts[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(nm)
        if not sm:
            return dict(sm_mhz=None, sm_max_mhz=None, reasons=["no samples"])
        return dict(sm_mhz=statistics.median(sm), sm_max_mhz=max(mx), reasons=sorted(reasons), samples=len(sm))


# =====================================================================================================
# CPU legs: the reference's native PyTorch path (or, if it cannot be imported, the numpy port)
# =====================================================================================================
def make_inputs_np(B, NH, S, DHQK, DHHV, seed):
    import numpy as np
    rng = np.random.default_rng(seed)
    out = dict(
        q=rng.standard_normal((B, NH, S, DHQK), dtype=np.float32),
        k=rng.standard_normal((B, NH, S, DHQK), dtype=np.float32),
        v=rng.standard_normal((B, NH, S, DHHV), dtype=np.float32),
        i=rng.standard_normal((B, NH, S), dtype=np.float32),
        f=3.0 + rng.standard_normal((B, NH, S), dtype=np.float32),
        dH=rng.standard_normal((B, NH, S, DHHV), dtype=np.float32),
    )
    return out


def import_reference_native():
    """The reference's native chunkwise function from the installed copy under baseline/_ref (or any importable
    mlstm_kernels).  Returns (function, None) or (None, reason)."""
    if os.path.isdir(REF_DIR) and REF_DIR not in sys.path:
        sys.path.insert(0, REF_DIR)
    try:
        from mlstm_kernels.torch.chunkwise.native.fwbw import mlstm_chunkwise__native_custbw
        return mlstm_chunkwise__native_custbw, None
    except Exception as e:  # noqa: BLE001
        return None, f"{type(e).__name__}: {e}"[:200]


def time_cpu_reference(steps, warmup):
    """(TFLOP/s, seconds per step, sample description, kind, threads) of the CPU leg."""
    import numpy as np
    w = WORKLOAD
    B, NH = CPU_SAMPLE["B"], CPU_SAMPLE["NH"]
    inp = make_inputs_np(B, NH, w["S"], w["DHQK"], w["DHHV"], seed=1)
    cores = os.cpu_count() or 1
    fn, why = import_reference_native()
    if fn is not None:
        import torch
        torch.set_num_threads(cores)
        t = {n: torch.from_numpy(x) for n, x in inp.items()}
        leaves = [t[n].clone().requires_grad_(True) for n in "qkvif"]

        def step():
            for x in leaves:
                x.grad = None
            H = fn(*leaves, chunk_size=w["L"])
            H.backward(t["dH"])
        kind, threads = "reference", torch.get_num_threads()
        what = "mlstm_chunkwise__native_custbw of the reference package (torch CPU, fp32)"
    else:
        from oracle import mlstm_oracle as O

        def step():
            O.chunkwise_fwbw(inp["q"], inp["k"], inp["v"], inp["i"], inp["f"], inp["dH"], chunk_size=w["L"],
                             dtype=np.float32)
        kind, threads = "port", cores
        what = f"numpy restatement of the reference's native path (reference not importable: {why})"

    def run():
        for _ in range(warmup):
            step()
        t0 = time.perf_counter()
        for _ in range(steps):
            step()
        return (time.perf_counter() - t0) / steps
    try:
        from threadpoolctl import threadpool_limits
        with threadpool_limits(limits=cores):
            dt = run()
    except ImportError:
        dt = run()
    fl = fw_flops(B, NH, w["S"], w["DHQK"], w["DHHV"], w["L"]) + bw_flops(B, NH, w["S"], w["DHQK"], w["DHHV"], w["L"])
    sample = (f"{what}; B={B} NH={NH} of the workload's B={w['B']} NH={w['NH']} (same S={w['S']}, head dims, chunk "
              f"size), {steps} timed steps of {dt:.2f} s, rate-normalised")
    return fl / dt / 1e12, dt, sample, kind, threads


def cpu_reference_small_cases():
    """The reference's own CPU code on the cases that fit a CPU: its native chunkwise function at BASELINE config 0
    (fp32, B=2, NH=4, S=512, 128/256, chunk 64; forward and forward+backward, 3 warm-up + 10 repetitions, median) and
    its native decode step (bf16 inputs, fp32 state, NH=8, 256/512; chained steps, per-step median)."""
    fn, why = import_reference_native()
    if fn is None:
        return {"unavailable": why}
    import torch
    from mlstm_kernels.torch.recurrent.native_step import mlstm_recurrent_step__native
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    out = {"cores": torch.get_num_threads()}
    B, NH, S, DHQK, DHHV, L = 2, 4, 512, 128, 256, 64
    g = torch.Generator().manual_seed(0)
    q, k, v = (torch.randn(B, NH, S, D, generator=g) for D in (DHQK, DHQK, DHHV))
    i, f, dH = torch.randn(B, NH, S, generator=g), 3 + torch.randn(B, NH, S, generator=g), torch.randn(B, NH, S, DHHV, generator=g)
    leaves = [t.clone().requires_grad_(True) for t in (q, k, v, i, f)]

    def med(fn_, reps, warm):
        for _ in range(warm):
            fn_()
        ts = []
        for _ in range(reps):
            t0 = time.perf_counter()
            fn_()
            ts.append(time.perf_counter() - t0)
        return statistics.median(ts)

    def fw():
        with torch.no_grad():
            fn(q, k, v, i, f, return_last_states=True, chunk_size=L)

    def fwbw():
        for t in leaves:
            t.grad = None
        fn(*leaves, return_last_states=True, chunk_size=L)[0].backward(dH)
    t_fw, t_fb = med(fw, 10, 3), med(fwbw, 10, 3)
    ffw = fw_flops(B, NH, S, DHQK, DHHV, L)
    ffb = ffw + bw_flops(B, NH, S, DHQK, DHHV, L)
    out["c0_chunkwise_native_custbw_fp32_B2_NH4_S512_128_256_L64"] = dict(
        fw_ms=t_fw * 1e3, fw_gflops=ffw / t_fw / 1e9, fwbw_ms=t_fb * 1e3, fwbw_gflops=ffb / t_fb / 1e9)
    NH, DHQK, DHHV = 8, 256, 512
    steps = {}
    for Bs, n in ((1, 16), (8, 16), (64, 16), (256, 4)):
        c, nn, m = 0.1 * torch.randn(Bs, NH, DHQK, DHHV, generator=g), torch.randn(Bs, NH, DHQK, generator=g).abs(), torch.randn(Bs, NH, 1, generator=g)
        tok = [tuple(torch.randn(Bs, NH, D, generator=g).bfloat16() for D in (DHQK, DHQK, DHHV)) +
               (torch.randn(Bs, NH, 1, generator=g).bfloat16(), (3 + torch.randn(Bs, NH, 1, generator=g)).bfloat16())
               for _ in range(n)]
        ts = []
        with torch.no_grad():
            for (qq, kk, vv, ii, ff) in tok:
                t0 = time.perf_counter()
                _, (c, nn, m) = mlstm_recurrent_step__native(qq, kk, vv, ii, ff, c, nn, m)
                ts.append(time.perf_counter() - t0)
        steps[f"B{Bs}"] = dict(ms_per_step=statistics.median(ts) * 1e3, tokens_per_s=Bs / statistics.median(ts))
    out["step_native_bf16_NH8_256_512"] = steps
    return out


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    val, dt, sample, kind, threads = time_cpu_reference(args.steps, args.warmup)
    w = WORKLOAD
    line = {
        "impl": "reference", "metric": METRIC, "value": val, "unit": "TFLOP/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": w["name"]},
        "cpu_baseline": {"value": val, "unit": "TFLOP/s", "cores": threads, "kind": kind, "sample": sample},
        "e2e": {"value": val, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line))


# =====================================================================================================
# GPU arm
# =====================================================================================================
def timed_local(torch, fn, steps, warmup):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / steps


def timed_reps(torch, fn, reps=30, warmup=10, flush=False):
    """The reference's timing protocol (mlstm_kernels/utils/benchmark/runtime.py:66-72,121-122): one CUDA-event pair
    per repetition, median (and min) over the repetitions; with `flush` a 256 MB buffer is zeroed before every
    repetition so that the L2 holds no input data."""
    cache = torch.empty(int(256e6 // 4), dtype=torch.int, device="cuda") if flush else None
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(reps)]
    for a, b in ev:
        if cache is not None:
            cache.zero_()
        a.record()
        fn()
        b.record()
    torch.cuda.synchronize()
    ts = [a.elapsed_time(b) for a, b in ev]
    return dict(median_ms=statistics.median(ts), min_ms=min(ts), reps=reps, warmup=warmup,
                l2_flush_256MB=bool(flush))


def prefer_gpu_numa_node(torch, index: int) -> dict:
    """Ask the kernel to place this thread's next allocations - the pinned host buffers of the end-to-end leg - on the
    NUMA node of its GPU (the PCI device's numa_node in sysfs; set_mempolicy(MPOL_PREFERRED)).  Memory placement only:
    CPU affinity and thread counts stay as they are.  Returns what was found and done (reported beside the end-to-end
    number); `default_memory_policy()` undoes it."""
    info = {"preferred_node_set": False}
    try:
        pr = torch.cuda.get_device_properties(index)
        bdf = f"{getattr(pr, 'pci_domain_id', 0):04x}:{pr.pci_bus_id:02x}:{pr.pci_device_id:02x}.0"
        with open(f"/sys/bus/pci/devices/{bdf}/numa_node") as fh:
            node = int(fh.read().strip())
        info["gpu_numa_node"] = node
        info["cpus_allowed"] = len(os.sched_getaffinity(0))
        if 0 <= node < 1024:
            import ctypes
            mask = (ctypes.c_ulong * 16)()
            mask[node // 64] = 1 << (node % 64)
            libc = ctypes.CDLL(None, use_errno=True)
            rc = libc.syscall(238, 1, mask, 1024)   # x86-64 set_mempolicy(MPOL_PREFERRED, mask, maxnode)
            info["preferred_node_set"] = rc == 0
            if rc != 0:
                info["note"] = f"set_mempolicy errno {ctypes.get_errno()}"
    except Exception as e:  # noqa: BLE001  (best effort: sysfs or the system call may be closed in a container)
        info["note"] = f"{type(e).__name__}: {e}"[:120]
    return info


def default_memory_policy() -> None:
    try:
        import ctypes
        ctypes.CDLL(None, use_errno=True).syscall(238, 0, None, 0)   # MPOL_DEFAULT
    except Exception:  # noqa: BLE001
        pass


def run_b200(args):
    import torch
    import torch.distributed as dist

    import mlstm_kernels_b200 as mk
    from mlstm_kernels_b200 import _lib

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world > 1:
        os.environ.setdefault("NCCL_NVLS_ENABLE", "0")   # point-to-point hand-offs only: no NVLink multicast binding
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    placement = prefer_gpu_numa_node(torch, local) if os.uname().machine == "x86_64" else {"preferred_node_set": False}
    w = WORKLOAD
    B, S, NH, DHQK, DHHV, L = (w[x] for x in ("B", "S", "NH", "DHQK", "DHHV", "L"))

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(x: float) -> float:
        if world == 1:
            return x
        t = torch.tensor([x], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    # ---- inputs: pinned host copies (for the end-to-end leg) and device-resident copies ----
    g = torch.Generator().manual_seed(1 + rank)
    host = {}
    for name, shape in (("q", (B, NH, S, DHQK)), ("k", (B, NH, S, DHQK)), ("v", (B, NH, S, DHHV)),
                        ("i", (B, NH, S)), ("f", (B, NH, S)), ("dH", (B, NH, S, DHHV))):
        t = torch.randn(shape, generator=g, dtype=torch.float32)
        if name == "f":
            t += 3.0
        host[name] = t.bfloat16().pin_memory()
    devin = {n: t.to(dev) for n, t in host.items()}
    leaf = {n: devin[n].clone().requires_grad_(True) for n in "qkvif"}
    RECOMPUTE = False   # the headline keeps the per-chunk states; the recompute setting is timed under `extra`

    def make_step(fn=None, recompute=RECOMPUTE, **kw):
        fn = fn or mk.mlstm_chunkwise__b200_xl_chunk

        def step():
            for t in leaf.values():
                t.grad = None
            H = fn(leaf["q"], leaf["k"], leaf["v"], leaf["i"], leaf["f"], chunk_size=L,
                   recompute_states_in_bw=recompute, **kw)
            H.backward(devin["dH"])
            return H
        return step

    step_resident = make_step()

    def fw_only():
        with torch.no_grad():
            return mk.mlstm_chunkwise__b200_xl_chunk(devin["q"], devin["k"], devin["v"], devin["i"], devin["f"],
                                                     chunk_size=L)

    host_out = {n: torch.empty_like(host[n]).pin_memory() for n in ("q", "k", "v", "i", "f")}
    host_out["H"] = torch.empty_like(host["v"]).pin_memory()
    default_memory_policy()   # the pinned buffers exist: later allocations go where the kernel likes again

    s_in, s_cmp, s_out = torch.cuda.Stream(), torch.cuda.Stream(), torch.cuda.Stream()

    # (batch, head) units are independent: the batch is fed in E2E_SLICES contiguous groups of units through two
    # preallocated sets of device staging buffers (no allocator traffic for the inputs inside the timed region)
    E2E_SLICES = args.e2e_slices
    units = B * NH
    per = units // E2E_SLICES
    hv = {n: t.view(1, units, *t.shape[2:]) for n, t in host.items()}
    hov = {n: t.view(1, units, *t.shape[2:]) for n, t in host_out.items()}
    stage = [{n: torch.empty((1, per, *t.shape[2:]), dtype=t.dtype, device=dev) for n, t in hv.items()} for _ in range(2)]

    def step_e2e():
        """Whole step from pinned host buffers to pinned host buffers through the public API.  The batch is fed in
        groups of (batch, head) units so that the H2D copy of group g+1, the kernels of group g and the D2H copy of
        group g-1 overlap (three streams); every byte still crosses PCIe inside the timed region."""
        cur = torch.cuda.current_stream()
        for st in (s_in, s_cmp, s_out):
            st.wait_stream(cur)
        consumed = [None, None]   # event: the kernels that read staging set j have finished
        for g in range(E2E_SLICES):
            sl = slice(g * per, (g + 1) * per)
            buf = stage[g % 2]
            with torch.cuda.stream(s_in):
                if consumed[g % 2] is not None:
                    s_in.wait_event(consumed[g % 2])
                for n in hv:
                    buf[n].copy_(hv[n][:, sl], non_blocking=True)
                ev_in = torch.cuda.Event()
                ev_in.record(s_in)
            with torch.cuda.stream(s_cmp):
                s_cmp.wait_event(ev_in)
                lf = {n: buf[n].detach().requires_grad_(True) for n in "qkvif"}
                H = mk.mlstm_chunkwise__b200_xl_chunk(lf["q"], lf["k"], lf["v"], lf["i"], lf["f"], chunk_size=L,
                                                      recompute_states_in_bw=RECOMPUTE)
                H.backward(buf["dH"])
                ev_c = torch.cuda.Event()
                ev_c.record(s_cmp)
                consumed[g % 2] = ev_c
            with torch.cuda.stream(s_out):
                s_out.wait_event(ev_c)
                outs = [("H", H.detach())] + [(n, lf[n].grad) for n in "qkvif"]
                for n, t in outs:
                    hov[n][:, sl].copy_(t, non_blocking=True)
                    t.record_stream(s_out)
        cur.wait_stream(s_cmp)
        cur.wait_stream(s_out)

    h2d = sum(t.numel() * t.element_size() for t in host.values())
    d2h = sum(t.numel() * t.element_size() for t in host_out.values())

    def timed(fn, steps, warmup):
        for _ in range(warmup):
            fn()
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            fn()
        e1.record()
        barrier()
        return max_over_ranks(e0.elapsed_time(e1) / steps)

    flops_fw = fw_flops(B, NH, S, DHQK, DHHV, L)
    flops_fwbw = flops_fw + bw_flops(B, NH, S, DHQK, DHHV, L)

    # ---- headline: fw+bw, inputs resident ----
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    n_before = _lib.launch_count()
    ms = timed(step_resident, args.steps, args.warmup)
    launches = (_lib.launch_count() - n_before) * args.steps // (args.steps + args.warmup)
    clocks = sampler.stop() if rank == 0 else None
    value = world * flops_fwbw / (ms * 1e-3) / 1e12

    if args.quick:
        if rank == 0:
            print(json.dumps({"metric": METRIC, "value": value, "unit": "TFLOP/s",
                              "ms_per_step": ms, "config": {"workload": w["name"]}, "quick": True}))
        if world > 1:
            dist.destroy_process_group()
        return

    # ---- end to end through the public API with host buffers ----
    e2e_steps = max(2, min(args.steps, 5))
    ms_e2e = timed(step_e2e, e2e_steps, 3)
    e2e_val = world * flops_fwbw / (ms_e2e * 1e-3) / 1e12

    # ---- per-kernel device time (CUDA events inside the library, on the launching stream) ----
    peaks = measured_peaks()
    impl_used = "tcgen05" if _lib.load().mlstm_b200_chunkwise_has_tcgen05(S, DHQK, DHHV, L, _lib.BF16) else "simt"

    def kernel_profile(step_fn, Bp, NHp, steps=5):
        _lib.profile_enable(True)
        for _ in range(steps):
            step_fn()
        torch.cuda.synchronize()
        prof = _lib.profile_read()
        _lib.profile_enable(False)
        pf = phase_flops(Bp, NHp, S, DHQK, DHHV, L)
        nchunks = Bp * NHp * (S // L)
        # the same kernels against the HBM roofline: algorithmic bytes per chunk (bf16 operands and states, outputs
        # written once; the figures listed next to the ncu capture in profiles/) divided by the measured time
        algo = {"recurrent_fw": 2 * L * (DHQK + DHHV) + 2 * DHQK * DHHV,
                "parallel_fw": 2 * L * (2 * DHQK + 2 * DHHV) + 2 * DHQK * DHHV,
                "recurrent_bw": 2 * L * (DHQK + DHHV) + 2 * DHQK * DHHV,
                "parallel_bw": 2 * L * (4 * DHQK + 3 * DHHV) + 4 * DHQK * DHHV}
        kernels = {}
        for name, (tot, cnt) in prof.items():
            if not cnt:
                continue
            kernels[name] = dict(ms=tot / cnt, launches_per_step=cnt / steps)
            if name in pf:
                kernels[name]["tflops"] = pf[name] / (tot / cnt * 1e-3) / 1e12
                gbs = algo[name] * nchunks / (tot / cnt * 1e-3) / 1e9
                kernels[name].update(hbm_gbs=gbs, hbm_frac=gbs / peaks["hbm"])
        return kernels

    kernels = kernel_profile(step_resident, B, NH, steps=max(2, min(args.steps, 5)))
    pf = phase_flops(B, NH, S, DHQK, DHHV, L)
    dom = max((n for n in kernels if n in pf), key=lambda n: kernels[n]["ms"] * kernels[n]["launches_per_step"])
    # DRAM bytes per launch of the dominant kernel: ncu dram__bytes_read.sum + dram__bytes_write.sum per chunk of 128
    # tokens, captured on a quarter batch (see profiles/), times the chunks of this launch (traffic is
    # proportional to the number of chunks)
    traffic = None
    if impl_used == "tcgen05" and (DHQK, DHHV, L) == (256, 256, 128) and dom in NCU_DRAM_BYTES_PER_CHUNK:
        traffic = NCU_DRAM_BYTES_PER_CHUNK[dom] * B * NH * (S // L)
    roofline = {"bound": "tensor", "kernel": dom, "achieved": kernels[dom]["tflops"], "peak": peaks["tflops"],
                "unit": "TFLOP/s", "frac": kernels[dom]["tflops"] / peaks["tflops"], "traffic": traffic,
                "peak_source": peaks["source"] + " (burst bf16 GEMM)", "impl": impl_used,
                "whole_step_frac": (flops_fwbw / (ms * 1e-3) / 1e12) / peaks["tflops"],
                "kernels": kernels}

    extra = {}
    # ---- multi-GPU blocks (every rank takes part; at N=1 they are the single-GPU figures) ----
    if not args.no_extra:
        extra["strong_scaling_fixed_batch"] = bench_strong(torch, dist, mk, _lib, dev, devin, world, rank, L, barrier,
                                                           max_over_ranks, kernel_profile, peaks)
        extra["step_decode_sharded_B256"] = bench_step_sharded(torch, mk, dev, world, rank, barrier, max_over_ranks,
                                                               peaks)
        extra["step_decode_sharded_B1_over_heads"] = bench_step_sharded(torch, mk, dev, world, rank, barrier,
                                                                        max_over_ranks, peaks, Btot=1)
        extra["sequence_parallel_prefill_B1_NH8_S131072_256_512_cs256"] = bench_sequence_parallel(
            torch, dist, mk, dev, world, rank, barrier, max_over_ranks, peaks)

    # ---- secondary single-GPU numbers (rank 0): forward only, recompute, mLSTMsig, protocol, decode, sweep ----
    if rank == 0 and not args.no_extra:
        ms_fw = timed_local(torch, fw_only, 5, 3)
        extra["fw_only"] = dict(ms=ms_fw, tflops=flops_fw / (ms_fw * 1e-3) / 1e12,
                                frac_of_peak=flops_fw / (ms_fw * 1e-3) / 1e12 / peaks["tflops"])

        def memory(recompute):
            """GB above the resident inputs: held between forward and backward, and at the peak of the step."""
            for t in leaf.values():
                t.grad = None
            torch.cuda.synchronize()
            torch.cuda.reset_peak_memory_stats()
            base = torch.cuda.memory_allocated()
            H = mk.mlstm_chunkwise__b200_xl_chunk(leaf["q"], leaf["k"], leaf["v"], leaf["i"], leaf["f"], chunk_size=L,
                                                  recompute_states_in_bw=recompute)
            torch.cuda.synchronize()
            held = torch.cuda.memory_allocated() - base
            H.backward(devin["dH"])
            torch.cuda.synchronize()
            peak = torch.cuda.max_memory_allocated() - base
            return dict(held_between_fw_and_bw_gb=held / 1e9, peak_gb=peak / 1e9)
        rec_step = make_step(recompute=True)
        ms_rec = timed_local(torch, rec_step, 5, 3)
        ms_keep = timed_local(torch, step_resident, 5, 3)
        extra["recompute_states_in_bw"] = {
            "False (headline setting)": dict(ms=ms_keep, tflops=flops_fwbw / (ms_keep * 1e-3) / 1e12, **memory(False)),
            "True (the reference's default)": dict(ms=ms_rec, tflops=flops_fwbw / (ms_rec * 1e-3) / 1e12,
                                                   **memory(True)),
            "note": "memory above the resident inputs (H and the input gradients included); timed back to back"}
        # the same step with every launch on one stream (the library's two-stream split of the units switched off)
        lib = _lib.load()
        prev_split = lib.mlstm_b200_set_unit_split(0)
        try:
            ms_one, ms_one_fw = timed_local(torch, step_resident, 5, 3), timed_local(torch, fw_only, 5, 3)
        finally:
            lib.mlstm_b200_set_unit_split(prev_split)
        ms_two, ms_two_fw = timed_local(torch, step_resident, 5, 3), timed_local(torch, fw_only, 5, 3)
        extra["two_stream_unit_split"] = {
            "on (default)": dict(fwbw_ms=ms_two, fw_ms=ms_two_fw), "off": dict(fwbw_ms=ms_one, fw_ms=ms_one_fw),
            "note": "when the recurrence's last wave of CTAs is poorly filled, the two halves of the (batch, head) "
                    "units run as two chains of launches on two streams; timed back to back"}
        sig_step = make_step(mk.mlstm_siging_chunkwise__b200_xl_chunk, normalize=True)
        ms_sig = timed_local(torch, sig_step, 5, 3)
        extra["fwbw_mLSTMsig"] = dict(ms=ms_sig, tflops=flops_fwbw / (ms_sig * 1e-3) / 1e12)
        # the reference's own protocol: >= 10 warm-up, 30 repetitions, median; with and without its 256 MB L2 flush
        extra["reference_protocol_fwbw"] = {
            "no_flush": timed_reps(torch, step_resident, 30, 10, flush=False),
            "l2_flush": timed_reps(torch, step_resident, 30, 10, flush=True)}
        extra["reference_protocol_fw"] = {
            "no_flush": timed_reps(torch, fw_only, 30, 10, flush=False),
            "l2_flush": timed_reps(torch, fw_only, 30, 10, flush=True)}
        extra["portable_kernels_f32_B4_NH4_S2048_64_128_L64"] = bench_portable(torch, mk, dev)
        extra["arbitrary_length_prefill_bf16_NH16_256_256"] = bench_any_length(torch, mk, dev)
        extra["head_dims_off_the_tile_bf16_B8_S8192"] = bench_head_dims(torch, mk, dev)
        extra["step_decode"] = bench_step(torch, mk, dev, peaks)
        extra["consttoken_sweep_65536_tokens"] = bench_sweep(torch, mk, dev, peaks)
        # the two head geometries of the reference's published constant-token figure (H100, its Triton kernels, median
        # with L2 flush: 6.36 ms forward / 15.2 ms fw+bw at NH=16 128/256; 8.2 / 20.7-21.2 ms at NH=8 256/512)
        extra["published_figure_geometries_65536_tokens"] = {
            "NH16_128_256": bench_sweep(torch, mk, dev, peaks, 16, 128, 256, ((8, 8192),)),
            "NH8_256_512": bench_sweep(torch, mk, dev, peaks, 8, 256, 512, ((8, 8192),)),
            "note": "same shapes as the reference's README figure (measured there on an H100 with its Triton kernels); "
                    "inputs follow this benchmark's distributions"}
        if world == 1 and not args.no_triton_ref:
            extra["reference_triton_same_gpu"] = bench_triton_reference(torch, devin, leaf, L, flops_fw, flops_fwbw)
    if world > 1:
        dist.barrier()

    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu:
        val, dt, sample, kind, threads = time_cpu_reference(5, 1)
        cpu = {"value": val, "unit": "TFLOP/s", "cores": threads, "kind": kind, "sample": sample}
        if not args.no_extra:
            try:
                extra["cpu_reference_small_cases"] = cpu_reference_small_cases()
            except Exception as e:  # noqa: BLE001  (a baseline for context must not take the GPU numbers down with it)
                extra["cpu_reference_small_cases"] = {"unavailable": f"{type(e).__name__}: {e}"[:200]}

    if rank == 0:
        line = {
            "metric": METRIC, "value": value, "unit": "TFLOP/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": w["name"]},
            "run": {"tokens_per_step_per_gpu": B * S, "tokens_per_s": world * B * S / (ms * 1e-3),
                    "sharding": "batch x heads, no collective; each rank runs its own batch (weak scaling); the fixed "
                                "batch split over the ranks is under extra.strong_scaling_fixed_batch",
                    "l2": "inputs (2.2 GB per step) larger than L2; no flush (a flushed variant is under "
                          "extra.reference_protocol_fwbw)",
                    "recompute_states_in_bw": RECOMPUTE, "impl": impl_used,
                    "streams": "two chains of launches (two halves of the units) when the recurrence's last wave is "
                               "poorly filled; extra.two_stream_unit_split times it on and off"},
            "roofline": roofline, "cpu_baseline": cpu,
            "e2e": {"value": e2e_val, "unit": "TFLOP/s", "ms_per_step": ms_e2e, "h2d_bytes_per_step": h2d,
                    "d2h_bytes_per_step": d2h,
                    "pcie_gbs_both_directions": (h2d + d2h) / (ms_e2e * 1e-3) / 1e9, "host_placement": placement},
            "gpu_launches": int(launches), "clocks": clocks, "extra": extra,
        }
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


def bench_strong(torch, dist, mk, _lib, dev, devin, world, rank, L, barrier, max_over_ranks, kernel_profile, peaks):
    """The FIXED benchmark batch (B=8 x NH=16 = 128 independent units) split contiguously over the ranks with
    shard_batch_heads: rank r runs 128 / N units, no collective on the data path.  Throughput = FLOPs of the whole
    batch / slowest rank's device time.  Every rank draws the same full batch (same seed) and slices its share."""
    from mlstm_kernels_b200.sharding import shard_batch_heads, shard_range
    w = WORKLOAD
    B, S, NH, DHQK, DHHV = (w[x] for x in ("B", "S", "NH", "DHQK", "DHHV"))
    g = torch.Generator(device=dev).manual_seed(11)
    full = {}
    for name, shape in (("q", (B, NH, S, DHQK)), ("k", (B, NH, S, DHQK)), ("v", (B, NH, S, DHHV)),
                        ("i", (B, NH, S)), ("f", (B, NH, S)), ("dH", (B, NH, S, DHHV))):
        t = torch.randn(shape, device=dev, generator=g)
        full[name] = (t + 3.0 if name == "f" else t).bfloat16()
    mine = dict(zip(full, shard_batch_heads(list(full.values()), world, rank)))
    del full
    lo, hi = shard_range(B * NH, world, rank)
    leaves = [mine[n].contiguous().clone().requires_grad_(True) for n in "qkvif"]
    dH = mine["dH"].contiguous()

    def step():
        for t in leaves:
            t.grad = None
        mk.mlstm_chunkwise__b200_xl_chunk(*leaves, chunk_size=L, recompute_states_in_bw=False).backward(dH)

    for _ in range(3):
        step()
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(10):
        step()
    e1.record()
    barrier()
    ms = max_over_ranks(e0.elapsed_time(e1) / 10)
    fl = fw_flops(B, NH, S, DHQK, DHHV, L) + bw_flops(B, NH, S, DHQK, DHHV, L)
    kern = kernel_profile(step, 1, hi - lo, steps=3)
    return dict(ms_per_step=ms, tflops=fl / (ms * 1e-3) / 1e12, tokens_per_s=B * S / (ms * 1e-3), n_gpus=world,
                units_total=B * NH, units_on_rank0=hi - lo, scaling="strong", collective="none",
                frac_of_n_gpu_peak=fl / (ms * 1e-3) / 1e12 / (world * peaks["tflops"]),
                kernels_rank0={k_: {x: v_[x] for x in ("ms", "tflops", "hbm_frac") if x in v_} for k_, v_ in kern.items()})


def bench_step_sharded(torch, mk, dev, world, rank, barrier, max_over_ranks, peaks, Btot=256):
    """Decode at NH=8, 256/512 with the batch sharded over the ranks (B / N sequences per rank, no collective):
    tokens/s of the whole batch = B / slowest rank's time per step.  A single sequence (B=1) cannot be split over the
    batch: its 8 heads are split over the ranks instead (launch-bound on any number of GPUs)."""
    from mlstm_kernels_b200.sharding import shard_range
    NH, DHQK, DHHV = 8, 256, 512
    if Btot == 1:
        lo, hi = shard_range(NH, min(world, NH), min(rank, NH - 1))
        Bm, NH = 1, hi - lo
    else:
        lo, hi = shard_range(Btot, world, rank)
        Bm = hi - lo
    g = torch.Generator(device=dev).manual_seed(100 + rank)
    c = torch.randn(Bm, NH, DHQK, DHHV, device=dev, generator=g) * 0.1
    n = torch.randn(Bm, NH, DHQK, device=dev, generator=g).abs()
    m = torch.randn(Bm, NH, 1, device=dev, generator=g)
    state = [(c, n, m), (torch.empty_like(c), torch.empty_like(n), torch.empty_like(m))]
    T = 32
    q, k = (torch.randn(T, Bm, NH, DHQK, device=dev, generator=g).bfloat16() for _ in range(2))
    v = torch.randn(T, Bm, NH, DHHV, device=dev, generator=g).bfloat16()
    i = torch.randn(T, Bm, NH, 1, device=dev, generator=g).bfloat16()
    f = (3 + torch.randn(T, Bm, NH, 1, device=dev, generator=g)).bfloat16()
    h = torch.empty(Bm, NH, DHHV, device=dev, dtype=torch.bfloat16)

    toks = [(q[t], k[t], v[t], i[t], f[t]) for t in range(T)]

    def run(nsteps):
        for t in range(nsteps):
            (ci, ni, mi), (co, no, mo) = state[t % 2], state[(t + 1) % 2]
            qt, kt, vt, it, ft = toks[t % T]
            mk.mlstm_recurrent_step__b200_fw(ci, ni, mi, qt, kt, vt, it, ft,
                                             matC_new=co, vecN_new=no, scaM_new=mo, vecH_out=h)
    nsteps = 256
    run(16)
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    run(nsteps)
    e1.record()
    barrier()
    us = max_over_ranks(e0.elapsed_time(e1) / nsteps * 1e3)
    gbs = step_bytes(Btot, 8, DHQK, DHHV) / (us * 1e-6) / 1e9
    return dict(us_per_step=us, tokens_per_s=Btot / (us * 1e-6), batch_total=Btot, batch_per_rank=Bm,
                heads_per_rank=NH, n_gpus=world, gbs_all_gpus=gbs, frac_of_n_gpu_hbm=gbs / (world * peaks["hbm"]),
                scaling="strong", collective="none")


def bench_sequence_parallel(torch, dist, mk, dev, world, rank, barrier, max_over_ranks, peaks):
    """Prefill of ONE long sequence (B=1, NH=8, 256/512, S=131072, requested chunk 256) with its chunks split
    contiguously over the ranks and the (C, n, m) boundary state handed from GPU to GPU (NCCL point-to-point, one
    message per hop).  Every rank draws the whole sequence from the same seed, runs the single-GPU pass as the
    reference result and its own segment through mlstm_chunkwise_sequence_parallel; times are device events, slowest
    rank.  FLOPs are counted at the chunk size the kernels actually run (128)."""
    from mlstm_kernels_b200.sharding import mlstm_chunkwise_sequence_parallel
    B, NH, S, DHQK, DHHV, Lreq = 1, 8, 131072, 256, 512, 256
    g = torch.Generator(device=dev).manual_seed(7)
    mk_t = lambda *sh: torch.randn(*sh, device=dev, generator=g).bfloat16()  # noqa: E731
    q, k, v = mk_t(B, NH, S, DHQK), mk_t(B, NH, S, DHQK), mk_t(B, NH, S, DHHV)
    i, f = mk_t(B, NH, S), (3 + torch.randn(B, NH, S, device=dev, generator=g)).bfloat16()
    dH = mk_t(B, NH, S, DHHV)
    Lrun = mk.kernel_chunk_size(q, v, Lreq)
    fl_fw = fw_flops(B, NH, S, DHQK, DHHV, Lrun)
    fl_fwbw = fl_fw + bw_flops(B, NH, S, DHQK, DHHV, Lrun)

    def single_fw():
        with torch.no_grad():
            return mk.mlstm_chunkwise__b200_xl_chunk(q, k, v, i, f, return_last_states=True, chunk_size=Lreq)
    ms_single = timed_local(torch, single_fw, 5, 3)
    out = dict(chunk_size_requested=Lreq, chunk_size_run=Lrun, n_gpus=world,
               single_gpu=dict(fw_ms=ms_single, fw_tflops=fl_fw / ms_single / 1e9,
                               fw_frac_of_peak=fl_fw / ms_single / 1e9 / peaks["tflops"],
                               tokens_per_s=S / (ms_single * 1e-3)))
    leaves = [t.clone().requires_grad_(True) for t in (q, k, v, i, f)]

    def single_fwbw():
        for t in leaves:
            t.grad = None
        mk.mlstm_chunkwise__b200_xl_chunk(*leaves, chunk_size=Lreq, recompute_states_in_bw=False).backward(dH)
    ms_single_fwbw = timed_local(torch, single_fwbw, 3, 2)
    out["single_gpu"].update(fwbw_ms=ms_single_fwbw, fwbw_tflops=fl_fwbw / ms_single_fwbw / 1e9)
    if world == 1:
        return out
    h_ref, last_ref = single_fw()
    grads_ref = [t.grad.clone() for t in leaves]
    seg = S // world
    sl = slice(rank * seg, (rank + 1) * seg)
    mine = [t[:, :, sl].contiguous() for t in (q, k, v, i, f)]
    dH_m = dH[:, :, sl].contiguous()

    def max_err(a, b):
        d = (a.float() - b.float()).abs().max() / b.float().abs().max().clamp_min(1e-30)
        return max_over_ranks(float(d))

    for mode in ("gather", "scan", "chain"):
        def sp_fw():
            with torch.no_grad():
                return mlstm_chunkwise_sequence_parallel(*mine, return_last_states=True, chunk_size=Lreq, mode=mode)
        for _ in range(2):
            sp_fw()
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(5):
            h_sp, last_sp = sp_fw()
        e1.record()
        barrier()
        ms = max_over_ranks(e0.elapsed_time(e1) / 5)
        res = dict(fw_ms=ms, fw_tflops=fl_fw / ms / 1e9, tokens_per_s=S / (ms * 1e-3),
                   speedup_vs_single_gpu=ms_single / ms,
                   H_max_rel_err_vs_single_gpu=max_err(h_sp, h_ref[:, :, sl]),
                   H_bit_identical=bool(max_over_ranks(0.0 if torch.equal(h_sp, h_ref[:, :, sl]) else 1.0) == 0.0),
                   C_last_max_rel_err=max_err(last_sp[0], last_ref[0]),
                   n_last_max_rel_err=max_err(last_sp[1], last_ref[1]),
                   m_last_max_abs_err=max_over_ranks(float((last_sp[2] - last_ref[2]).abs().max())))
        # forward + backward (gather, scan: the segments' backwards run concurrently; chain: right to left)
        lv = [t.clone().requires_grad_(True) for t in mine]

        def sp_fwbw():
            for t in lv:
                t.grad = None
            mlstm_chunkwise_sequence_parallel(*lv, chunk_size=Lreq, mode=mode).backward(dH_m)
        sp_fwbw()
        barrier()
        e0.record()
        for _ in range(3):
            sp_fwbw()
        e1.record()
        barrier()
        msb = max_over_ranks(e0.elapsed_time(e1) / 3)
        res.update(fwbw_ms=msb, fwbw_tflops=fl_fwbw / msb / 1e9, fwbw_speedup_vs_single_gpu=ms_single_fwbw / msb)
        for name, a, b in zip(("dQ", "dK", "dV", "dI", "dF"), lv, grads_ref):
            res[f"{name}_max_rel_err_vs_single_gpu"] = max_err(a.grad, b[:, :, sl])
        out[mode] = res
    out["exchange"] = ("gather: one NCCL all-gather of the packed segment summaries (forward) and of the packed "
                       "(dC_own, decay) pairs (backward), folded locally in rank order; scan / chain: (C, n, m) packed "
                       "into one NCCL point-to-point message per hop (4.2 MB); segments concurrent in gather and scan")
    return out


def bench_triton_reference(torch, devin, leaf, L, flops_fw, flops_fwbw):
    """The reference's own Triton kernels, JIT-compiled by the machine's Triton, on the same GPU, inputs and timing
    loop (the first calls, which compile, are excluded).  Needs the reference package to be importable (e.g.
    pip-installed with --target baseline/_ref); reports the error text otherwise."""
    if os.path.isdir(REF_DIR) and REF_DIR not in sys.path:
        sys.path.insert(0, REF_DIR)
    out = {}
    try:
        from mlstm_kernels.torch.chunkwise.triton_xl_chunk import mlstm_chunkwise__xl_chunk
        from mlstm_kernels.torch.chunkwise.triton_xl_chunk_siging import mlstm_siging_chunkwise__xl_chunk
    except Exception as e:  # noqa: BLE001
        return {"unavailable": f"{type(e).__name__}: {e}"[:300]}

    def make(fn, **kw):
        def step():
            for t in leaf.values():
                t.grad = None
            H = fn(leaf["q"], leaf["k"], leaf["v"], leaf["i"], leaf["f"], chunk_size=L, **kw)
            H.backward(devin["dH"])
        return step

    def fw_only():
        with torch.no_grad():
            mlstm_chunkwise__xl_chunk(devin["q"], devin["k"], devin["v"], devin["i"], devin["f"], chunk_size=L)

    for name, fn, fl in (("fwbw_mLSTMexp_recompute_states (its default)", make(mlstm_chunkwise__xl_chunk), flops_fwbw),
                         ("fwbw_mLSTMexp_keep_states", make(mlstm_chunkwise__xl_chunk, recompute_states_in_bw=False), flops_fwbw),
                         ("fw_mLSTMexp", fw_only, flops_fw),
                         ("fwbw_mLSTMsig_recompute_states (its default)", make(mlstm_siging_chunkwise__xl_chunk, normalize=True), flops_fwbw)):
        try:
            ms = timed_local(torch, fn, 5, 3)
            torch.cuda.synchronize()
            torch.cuda.reset_peak_memory_stats()
            base = torch.cuda.memory_allocated()
            fn()
            torch.cuda.synchronize()
            out[name] = dict(ms=ms, tflops=fl / (ms * 1e-3) / 1e12,
                             peak_extra_memory_gb=(torch.cuda.max_memory_allocated() - base) / 1e9)
        except Exception as e:  # noqa: BLE001
            out[name] = {"unavailable": f"{type(e).__name__}: {e}"[:300]}
    try:   # arbitrary-length prefill through the reference's own wrapper (chunk-size ladder + per-token tail loop)
        from mlstm_kernels.torch.backend_module import mLSTMBackend, mLSTMBackendConfig
        backend = mLSTMBackend(mLSTMBackendConfig(chunkwise_kernel="chunkwise--triton_xl_chunk",
                                                   sequence_kernel="native_sequence__triton", step_kernel="triton",
                                                   mode="inference", chunk_size=128, return_last_states=True,
                                                   autocast_kernel_dtype="bfloat16", inference_state_dtype="float32"))
        dev = devin["q"].device
        for B, S in ((8, 500), (8, 8000 + 77)):
            g = torch.Generator(device=dev).manual_seed(S)
            mk_t = lambda *sh: torch.randn(*sh, device=dev, generator=g).bfloat16()  # noqa: E731
            q, k, v = mk_t(B, 16, S, 256), mk_t(B, 16, S, 256), mk_t(B, 16, S, 256)
            i, f = mk_t(B, 16, S), (3 + torch.randn(B, 16, S, device=dev, generator=g)).bfloat16()

            def fw():
                with torch.no_grad():
                    backend(q, k, v, i, f)
            ms = timed_local(torch, fw, 5, 3)
            out[f"arbitrary_length_prefill_B{B}_S{S}"] = dict(fw_ms=ms, tokens_per_s=B * S / (ms * 1e-3))
    except Exception as e:  # noqa: BLE001
        out["arbitrary_length_prefill"] = {"unavailable": f"{type(e).__name__}: {e}"[:300]}
    try:
        from mlstm_kernels.torch.recurrent.triton_step import mlstm_recurrent_step__triton
        NH, DHQK, DHHV = 8, 256, 512
        dev = devin["q"].device
        for B in (1, 8, 64, 256):
            c = torch.randn(B, NH, DHQK, DHHV, device=dev) * 0.1
            n = torch.randn(B, NH, DHQK, device=dev).abs()
            m = torch.randn(B, NH, 1, device=dev)
            q = torch.randn(B, NH, DHQK, device=dev).bfloat16(); k = torch.randn_like(q)
            v = torch.randn(B, NH, DHHV, device=dev).bfloat16()
            i = torch.randn(B, NH, 1, device=dev).bfloat16(); f = (3 + torch.randn(B, NH, 1, device=dev)).bfloat16()
            fn = lambda: mlstm_recurrent_step__triton(q, k, v, i, f, c, n, m)  # noqa: E731
            ms = timed_local(torch, fn, 200 if B <= 64 else 50, 10)
            out[f"step_B{B}"] = dict(us_per_step=ms * 1e3, tokens_per_s=B / (ms * 1e-3))
    except Exception as e:  # noqa: BLE001
        out["step"] = {"unavailable": f"{type(e).__name__}: {e}"[:300]}
    return out


def bench_portable(torch, mk, dev):
    """The CUDA-core kernels that take every case the tcgen05 path does not (f32 inputs, head dims that are no
    multiples of 8): one f32 case in the reference's own test geometry, forward and forward+backward."""
    B, NH, S, DHQK, DHHV, L = 4, 4, 2048, 64, 128, 64
    g = torch.Generator(device=dev).manual_seed(3)
    mk_t = lambda *sh: torch.randn(*sh, device=dev, generator=g)  # noqa: E731
    q, k, v, i, f, dH = mk_t(B, NH, S, DHQK), mk_t(B, NH, S, DHQK), mk_t(B, NH, S, DHHV), mk_t(B, NH, S), 3 + mk_t(B, NH, S), mk_t(B, NH, S, DHHV)
    leaf = [t.clone().requires_grad_(True) for t in (q, k, v, i, f)]

    def fw():
        with torch.no_grad():
            mk.mlstm_chunkwise__b200_xl_chunk(q, k, v, i, f, chunk_size=L)

    def fwbw():
        for t in leaf:
            t.grad = None
        mk.mlstm_chunkwise__b200_xl_chunk(*leaf, chunk_size=L).backward(dH)
    ms_fw, ms_fwbw = timed_local(torch, fw, 5, 3), timed_local(torch, fwbw, 5, 3)
    ffw = fw_flops(B, NH, S, DHQK, DHHV, L)
    ffb = ffw + bw_flops(B, NH, S, DHQK, DHHV, L)
    return dict(fw_ms=ms_fw, fw_tflops=ffw / ms_fw / 1e9, fwbw_ms=ms_fwbw, fwbw_tflops=ffb / ms_fwbw / 1e9,
                note="exact f32 arithmetic on CUDA cores (coverage path, not tuned)")


def bench_head_dims(torch, mk, dev):
    """Head dims that are no multiples of the kernels' 128-wide tiles (small-model geometries), bf16, B=8, S=8192: the
    tcgen05 path pads the tiles with zeros inside TMA; the same call on the CUDA-core kernels beside it."""
    out = {}
    for NH, DHQK, DHHV in ((4, 96, 192), (8, 64, 128), (4, 192, 384)):
        B, S = 8, 8192
        g = torch.Generator(device=dev).manual_seed(DHQK)
        mk_t = lambda *sh: torch.randn(*sh, device=dev, generator=g).bfloat16()  # noqa: E731
        q, k, v, dH = mk_t(B, NH, S, DHQK), mk_t(B, NH, S, DHQK), mk_t(B, NH, S, DHHV), mk_t(B, NH, S, DHHV)
        i, f = mk_t(B, NH, S), (3 + torch.randn(B, NH, S, device=dev, generator=g)).bfloat16()
        leaf = [t.clone().requires_grad_(True) for t in (q, k, v, i, f)]
        ffw = fw_flops(B, NH, S, DHQK, DHHV, 128)
        ffb = ffw + bw_flops(B, NH, S, DHQK, DHHV, 128)
        res = {}
        for impl, reps in (("auto", 10), ("simt", 3)):
            def fwbw():
                for t in leaf:
                    t.grad = None
                mk.mlstm_chunkwise__b200_xl_chunk(*leaf, chunk_size=128, impl=impl).backward(dH)
            ms = timed_local(torch, fwbw, reps, 3)
            res["tcgen05" if impl == "auto" else "cuda_cores"] = dict(fwbw_ms=ms, fwbw_tflops=ffb / ms / 1e9)
        out[f"NH{NH}_{DHQK}_{DHHV}"] = res
    return out


def bench_any_length(torch, mk, dev):
    """Prefill (forward with last states) of sequences whose length is no multiple of the chunk size, bf16, NH=16,
    256/256, B=8: one call on the tcgen05 path with a ragged last chunk; no host-side padding, no chunk-size ladder."""
    NH, DHQK, DHHV = 16, 256, 256
    out = {}
    for B, S in ((8, 500), (8, 8000 + 77)):
        g = torch.Generator(device=dev).manual_seed(S)
        mk_t = lambda *sh: torch.randn(*sh, device=dev, generator=g).bfloat16()  # noqa: E731
        q, k, v = mk_t(B, NH, S, DHQK), mk_t(B, NH, S, DHQK), mk_t(B, NH, S, DHHV)
        i, f = mk_t(B, NH, S), (3 + torch.randn(B, NH, S, device=dev, generator=g)).bfloat16()

        def fw():
            with torch.no_grad():
                mk.mlstm_chunkwise__b200_xl_chunk(q, k, v, i, f, return_last_states=True, chunk_size=128)
        ms = timed_local(torch, fw, 10, 3)
        fl = fw_flops(B, NH, S, DHQK, DHHV, 128)
        out[f"B{B}_S{S}"] = dict(fw_ms=ms, fw_tflops=fl / ms / 1e9, tokens_per_s=B * S / (ms * 1e-3))
    return out


def bench_sweep(torch, mk, dev, peaks, NH=16, DHQK=256, DHHV=256, points=((128, 512), (64, 1024), (32, 2048),
                                                                            (16, 4096), (8, 8192), (4, 16384))):
    """The baseline's constant-token sweep (65,536 tokens, NH=16, 256/256, chunk 128, bf16): forward and
    forward+backward for mLSTMexp at every (B, S) point.  Other head geometries on request."""
    L = 128
    out = {}
    for B, S in points:
        g = torch.Generator(device=dev).manual_seed(S)
        mk_t = lambda *sh: torch.randn(*sh, device=dev, generator=g).bfloat16()  # noqa: E731
        q, k, v = mk_t(B, NH, S, DHQK), mk_t(B, NH, S, DHQK), mk_t(B, NH, S, DHHV)
        i, f = mk_t(B, NH, S), (3 + torch.randn(B, NH, S, device=dev, generator=g)).bfloat16()
        dH = mk_t(B, NH, S, DHHV)
        leaf = [t.clone().requires_grad_(True) for t in (q, k, v, i, f)]

        def fw():
            with torch.no_grad():
                mk.mlstm_chunkwise__b200_xl_chunk(q, k, v, i, f, chunk_size=L)

        def fwbw():
            for t in leaf:
                t.grad = None
            mk.mlstm_chunkwise__b200_xl_chunk(*leaf, chunk_size=L, recompute_states_in_bw=False).backward(dH)
        ms_fw, ms_fwbw = timed_local(torch, fw, 5, 3), timed_local(torch, fwbw, 5, 3)
        ffw = fw_flops(B, NH, S, DHQK, DHHV, L)
        ffb = ffw + bw_flops(B, NH, S, DHQK, DHHV, L)
        out[f"B{B}_S{S}"] = dict(fw_ms=ms_fw, fw_tflops=ffw / ms_fw / 1e9, fw_frac_of_peak=ffw / ms_fw / 1e9 / peaks["tflops"],
                                 fwbw_ms=ms_fwbw, fwbw_tflops=ffb / ms_fwbw / 1e9,
                                 fwbw_frac_of_peak=ffb / ms_fwbw / 1e9 / peaks["tflops"])
        del q, k, v, i, f, dH, leaf
    return out


def bench_step(torch, mk, dev, peaks):
    """Decode at the xLSTM-7B head geometry NH=8, 256/512, bf16 tokens, f32 state; chained steps."""
    NH, DHQK, DHHV = 8, 256, 512
    out = {}
    for B in (1, 8, 64, 256):
        g = torch.Generator(device=dev).manual_seed(B)
        c = torch.randn(B, NH, DHQK, DHHV, device=dev, generator=g) * 0.1
        n = torch.randn(B, NH, DHQK, device=dev, generator=g).abs()
        m = torch.randn(B, NH, 1, device=dev, generator=g)
        c2, n2, m2 = torch.empty_like(c), torch.empty_like(n), torch.empty_like(m)
        T = 64
        q = torch.randn(T, B, NH, DHQK, device=dev, generator=g).bfloat16()
        k = torch.randn(T, B, NH, DHQK, device=dev, generator=g).bfloat16()
        v = torch.randn(T, B, NH, DHHV, device=dev, generator=g).bfloat16()
        i = torch.randn(T, B, NH, 1, device=dev, generator=g).bfloat16()
        f = (3 + torch.randn(T, B, NH, 1, device=dev, generator=g)).bfloat16()
        h = torch.empty(B, NH, DHHV, device=dev, dtype=torch.bfloat16)
        state = [(c, n, m), (c2, n2, m2)]

        # per-step token tensors are sliced ahead of the loop (a decoder gets them from its projection layers)
        toks = [(q[t], k[t], v[t], i[t], f[t]) for t in range(T)]

        def run(nsteps):
            for t in range(nsteps):
                (ci, ni, mi), (co, no, mo) = state[t % 2], state[(t + 1) % 2]
                qt, kt, vt, it, ft = toks[t % T]
                mk.mlstm_recurrent_step__b200_fw(ci, ni, mi, qt, kt, vt, it, ft,
                                                 matC_new=co, vecN_new=no, scaM_new=mo, vecH_out=h)
        nsteps = 1024 if B <= 64 else 256
        run(16)
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        run(nsteps)
        e1.record()
        torch.cuda.synchronize()
        us = e0.elapsed_time(e1) / nsteps * 1e3
        nbytes = step_bytes(B, NH, DHQK, DHHV)
        gbs = nbytes / (us * 1e-6) / 1e9
        out[f"B{B}"] = dict(us_per_step=us, tokens_per_s=B / (us * 1e-6), gbs=gbs, frac_of_hbm=gbs / peaks["hbm"],
                            note="includes Python launch overhead per step" if B <= 8 else "")
        if B <= 8:
            # decode loop that owns all its buffers: argument validation and conversions switched off
            def run_fast(nsteps):
                for t in range(nsteps):
                    (ci, ni, mi), (co, no, mo) = state[t % 2], state[(t + 1) % 2]
                    qt, kt, vt, it, ft = toks[t % T]
                    mk.mlstm_recurrent_step__b200_fw(ci, ni, mi, qt, kt, vt, it, ft, matC_new=co, vecN_new=no,
                                                     scaM_new=mo, vecH_out=h, validate=False)
            run_fast(16)
            torch.cuda.synchronize()
            e0.record()
            run_fast(nsteps)
            e1.record()
            torch.cuda.synchronize()
            us_f = e0.elapsed_time(e1) / nsteps * 1e3
            out[f"B{B}"].update(us_per_step_validate_off=us_f, tokens_per_s_validate_off=B / (us_f * 1e-6))
            # the same chain of steps captured once in a CUDA graph and replayed: device time without the host loop
            side = torch.cuda.Stream()
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                run(2)
            torch.cuda.current_stream().wait_stream(side)
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                run(T)
            graph.replay()
            torch.cuda.synchronize()
            e0.record()
            for _ in range(16):
                graph.replay()
            e1.record()
            torch.cuda.synchronize()
            us_g = e0.elapsed_time(e1) / (16 * T) * 1e3
            out[f"B{B}"].update(us_per_step_cuda_graph=us_g, tokens_per_s_cuda_graph=B / (us_g * 1e-6),
                                gbs_cuda_graph=nbytes / (us_g * 1e-6) / 1e9,
                                note_cuda_graph="both state buffers of this batch size fit the 126 MB L2")
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--no-extra", action="store_true", help="skip the secondary measurements")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--no-triton-ref", action="store_true",
                    help="do not time the reference's Triton kernels on this GPU (they run by default at N=1 when the "
                         "reference package is importable)")
    ap.add_argument("--e2e-slices", type=int, default=8,
                    help="groups of (batch, head) units the end-to-end leg pipelines over PCIe (must divide B*NH)")
    ap.add_argument("--batch", type=int, default=None, help="override the batch size B of the workload (profiling)")
    ap.add_argument("--quick", action="store_true",
                    help="profiling mode: timed region only (no end-to-end leg, no per-kernel pass, no extras, no CPU leg)")
    ap.add_argument("--step-only", type=int, default=None, metavar="B",
                    help="profiling mode: a short chain of decode steps at batch B (NH=8, 256/512) and nothing else")
    args = ap.parse_args()
    if args.warmup < 3 and args.impl == "b200" and not args.quick:
        args.warmup = 3
    if args.batch is not None:
        WORKLOAD["B"] = args.batch
        WORKLOAD["name"] = WORKLOAD["name"].replace("_B8_", f"_B{args.batch}_")
    if args.quick:
        args.no_extra = args.no_cpu = True
    if args.step_only is not None:
        run_step_only(args.step_only)
    elif args.impl == "reference":
        run_reference(args)
    else:
        run_b200(args)


def run_step_only(B):
    """A chain of 24 decode steps at batch B, for a profiler capture of the decode kernel alone."""
    import torch

    import mlstm_kernels_b200 as mk
    dev = torch.device("cuda", 0)
    NH, DHQK, DHHV = 8, 256, 512
    c = torch.randn(B, NH, DHQK, DHHV, device=dev) * 0.1
    n = torch.randn(B, NH, DHQK, device=dev).abs()
    m = torch.randn(B, NH, 1, device=dev)
    state = [(c, n, m), (torch.empty_like(c), torch.empty_like(n), torch.empty_like(m))]
    q, k = torch.randn(B, NH, DHQK, device=dev).bfloat16(), torch.randn(B, NH, DHQK, device=dev).bfloat16()
    v = torch.randn(B, NH, DHHV, device=dev).bfloat16()
    i, f = torch.randn(B, NH, 1, device=dev).bfloat16(), (3 + torch.randn(B, NH, 1, device=dev)).bfloat16()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    for t in range(24):
        if t == 8:
            e0.record()
        (ci, ni, mi), (co, no, mo) = state[t % 2], state[(t + 1) % 2]
        mk.mlstm_recurrent_step__b200_fw(ci, ni, mi, q, k, v, i, f, matC_new=co, vecN_new=no, scaM_new=mo)
    e1.record()
    torch.cuda.synchronize()
    us = e0.elapsed_time(e1) / 16 * 1e3
    print(json.dumps({"step_only_B": B, "us_per_step": us, "gbs": step_bytes(B, NH, DHQK, DHHV) / (us * 1e-6) / 1e9}))


if __name__ == "__main__":
    main()
