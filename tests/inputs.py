"""Seeded synthetic inputs shared by the golden-vector generator and the tests.

numpy's PCG64 stream is platform independent, so the golden generator and every test (on
any machine) see bit-identical inputs.  Distributions: q, k, v, i ~ N(0,1); f = f_offset + N(0,1)
(pre-log-sigmoid forget logits); upstream gradient dH ~ N(0,1); decode states
C ~ N(0, 0.1), n ~ |N(0,1)|, m ~ N(0,1).
"""

from __future__ import annotations

import numpy as np

# name -> case description.  `stride` > 1 stores / compares every stride-th element of the
# flattened arrays (keeps the big fixture small).
CASES = {
    # the reference's own test shape (tests/conftest.py final_combinations) at chunk size 64
    "exp_small": dict(kind="exp_chunkwise", seed=0, B=1, NH=2, S=256, DHQK=64, DHHV=128, L=64, f_offset=3.0),
    # initial states + incoming dC_last, small odd-ish dims
    "exp_init": dict(kind="exp_chunkwise", seed=1, B=2, NH=2, S=128, DHQK=32, DHHV=64, L=32, f_offset=3.0,
                     init=True, dC_last=True),
    # forget logits without offset: strong decay, exercises the stabiliser
    "exp_decay": dict(kind="exp_chunkwise", seed=2, B=1, NH=2, S=256, DHQK=32, DHHV=32, L=128, f_offset=0.0),
    # CPU-runnable configuration of the baseline: B=2 NH=4 S=512 128/256 L=64
    "exp_c0": dict(kind="exp_chunkwise", seed=0, B=2, NH=4, S=512, DHQK=128, DHHV=256, L=64, f_offset=3.0, stride=31),
    # quadratic secondary oracle for mLSTMexp
    "exp_parallel": dict(kind="exp_parallel", seed=0, B=1, NH=2, S=256, DHQK=64, DHHV=128, L=64, f_offset=3.0),
    # mLSTMsig: the quadratic formulation is the reference's only native implementation
    "sig_norm": dict(kind="sig_parallel", seed=3, B=1, NH=2, S=256, DHQK=64, DHHV=128, L=64, f_offset=3.0,
                     normalize=True),
    "sig_nonorm": dict(kind="sig_parallel", seed=4, B=1, NH=2, S=256, DHQK=64, DHHV=128, L=64, f_offset=3.0,
                       normalize=False),
    # mLSTMsig final states (C, n) read out of the reference's quadratic implementation with probe tokens
    "sig_states": dict(kind="sig_states", seed=6, B=1, NH=2, S=256, DHQK=64, DHHV=128, L=64, f_offset=3.0),
    # decode: 4 chained steps
    "step_small": dict(kind="step", seed=5, B=2, NH=4, DHQK=64, DHHV=128, steps=4, f_offset=3.0),
}


def make_chunkwise_inputs(case: dict, dtype=np.float32) -> dict:
    rng = np.random.default_rng(case["seed"])
    B, NH, S, DHQK, DHHV = (case[n] for n in ("B", "NH", "S", "DHQK", "DHHV"))
    out = {}
    out["q"] = rng.standard_normal((B, NH, S, DHQK), dtype=np.float32)
    out["k"] = rng.standard_normal((B, NH, S, DHQK), dtype=np.float32)
    out["v"] = rng.standard_normal((B, NH, S, DHHV), dtype=np.float32)
    out["i"] = rng.standard_normal((B, NH, S), dtype=np.float32)
    out["f"] = (case.get("f_offset", 3.0) + rng.standard_normal((B, NH, S), dtype=np.float32)).astype(np.float32)
    out["dH"] = rng.standard_normal((B, NH, S, DHHV), dtype=np.float32)
    if case.get("init"):
        out["c0"] = (0.1 * rng.standard_normal((B, NH, DHQK, DHHV), dtype=np.float32)).astype(np.float32)
        out["n0"] = np.abs(rng.standard_normal((B, NH, DHQK), dtype=np.float32))
        out["m0"] = rng.standard_normal((B, NH, 1), dtype=np.float32)
    if case.get("dC_last"):
        out["dC_last"] = rng.standard_normal((B, NH, DHQK, DHHV), dtype=np.float32)
    return {n: x.astype(dtype) for n, x in out.items()}


def make_step_inputs(case: dict, dtype=np.float32) -> dict:
    rng = np.random.default_rng(case["seed"])
    B, NH, DHQK, DHHV, T = (case[n] for n in ("B", "NH", "DHQK", "DHHV", "steps"))
    out = {}
    out["c"] = (0.1 * rng.standard_normal((B, NH, DHQK, DHHV), dtype=np.float32)).astype(np.float32)
    out["n"] = np.abs(rng.standard_normal((B, NH, DHQK), dtype=np.float32))
    out["m"] = rng.standard_normal((B, NH, 1), dtype=np.float32)
    out["q"] = rng.standard_normal((T, B, NH, DHQK), dtype=np.float32)
    out["k"] = rng.standard_normal((T, B, NH, DHQK), dtype=np.float32)
    out["v"] = rng.standard_normal((T, B, NH, DHHV), dtype=np.float32)
    out["i"] = rng.standard_normal((T, B, NH, 1), dtype=np.float32)
    out["f"] = (case.get("f_offset", 3.0) + rng.standard_normal((T, B, NH, 1), dtype=np.float32)).astype(np.float32)
    return {n: x.astype(dtype) for n, x in out.items()}


def subsample(x: np.ndarray, stride: int) -> np.ndarray:
    """Every stride-th element of the flattened array (identity for stride 1)."""
    if stride <= 1:
        return x
    return np.ascontiguousarray(x.reshape(-1)[::stride])


def max_rel_err(a: np.ndarray, b: np.ndarray) -> float:
    """max |a-b| / max |b|: the normalised maximum error used for the stated tolerances."""
    a = np.asarray(a, np.float64); b = np.asarray(b, np.float64)
    return float(np.abs(a - b).max() / max(np.abs(b).max(), 1e-30))


def elementwise_ok_fraction(a: np.ndarray, b: np.ndarray, rtol: float, atol: float) -> float:
    """Fraction of elements with |a - b| <= rtol * |b| + atol."""
    a = np.asarray(a, np.float64); b = np.asarray(b, np.float64)
    return float(np.mean(np.abs(a - b) <= rtol * np.abs(b) + atol))


def rms(x: np.ndarray) -> float:
    x = np.asarray(x, np.float64)
    return float(np.sqrt(np.mean(x * x)))
