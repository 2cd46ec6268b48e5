"""Pins the numpy oracle to the reference: every oracle function is compared with outputs of
the reference's own PyTorch implementation stored in tests/golden (see make_golden.py)."""

import os

import numpy as np
import pytest

from inputs import CASES, make_chunkwise_inputs, make_step_inputs, max_rel_err, subsample
from oracle import mlstm_oracle as O

GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")

# fp32 reference vs float64 oracle: normalised max error
TOL_FW = 2e-5
TOL_BW = 2e-4


def load(name):
    return dict(np.load(os.path.join(GOLD, f"{name}.npz")))


@pytest.mark.parametrize("name", [n for n, c in CASES.items() if c["kind"] == "exp_chunkwise"])
def test_exp_chunkwise_matches_reference(name):
    case, gold = CASES[name], load(name)
    inp = make_chunkwise_inputs(case)
    fw, bw = O.chunkwise_fwbw(
        inp["q"], inp["k"], inp["v"], inp["i"], inp["f"], inp["dH"],
        c_initial=inp.get("c0"), n_initial=inp.get("n0"), m_initial=inp.get("m0"), dC_last=inp.get("dC_last"),
        chunk_size=case["L"], eps=1e-6)
    st = case.get("stride", 1)
    for key in ("H", "n_out", "m_out", "C_last", "n_last", "m_last", "C_states", "n_states", "m_states"):
        assert max_rel_err(subsample(fw[key], st), gold[key]) < TOL_FW, key
    for key in ("dQ", "dK", "dV", "dI", "dF"):
        assert max_rel_err(subsample(bw[key], st), gold[key]) < TOL_BW, key
    if "dC_initial" in gold:
        assert max_rel_err(subsample(bw["dC_initial"], st), gold["dC_initial"]) < TOL_BW


def test_exp_chunkwise_matches_reference_parallel():
    """Secondary oracle: the quadratic stabilised formulation (what the reference's own tests compare with)."""
    case, gold = CASES["exp_parallel"], load("exp_parallel")
    inp = make_chunkwise_inputs(case)
    fw, bw = O.chunkwise_fwbw(inp["q"], inp["k"], inp["v"], inp["i"], inp["f"], inp["dH"], chunk_size=case["L"])
    assert max_rel_err(fw["H"], gold["H"]) < TOL_FW
    for key in ("dQ", "dK", "dV", "dI", "dF"):
        assert max_rel_err(bw[key], gold[key]) < TOL_BW, key


@pytest.mark.parametrize("name", ["sig_norm", "sig_nonorm"])
@pytest.mark.parametrize("L", [64, 128])
def test_sig_chunkwise_matches_reference_parallel(name, L):
    case, gold = CASES[name], load(name)
    inp = make_chunkwise_inputs(case)
    fw, bw = O.chunkwise_fwbw(inp["q"], inp["k"], inp["v"], inp["i"], inp["f"], inp["dH"], chunk_size=L,
                              siging=True, normalize=case["normalize"])
    assert max_rel_err(fw["H"], gold["H"]) < TOL_FW
    for key in ("dQ", "dK", "dV", "dI", "dF"):
        assert max_rel_err(bw[key], gold[key]) < TOL_BW, key
    H2 = O.parallel_siging_fw(inp["q"], inp["k"], inp["v"], inp["i"], inp["f"], normalize=case["normalize"])
    assert max_rel_err(H2, gold["H"]) < TOL_FW


@pytest.mark.parametrize("L", [32, 64, 256])
def test_siging_states_match_reference(L):
    """The oracle's mLSTMsig final state (C, n) against values read out of the reference's quadratic implementation
    through probe tokens (tests/golden/make_golden.py:run_sig_states); independent of the chunk size."""
    case, gold = CASES["sig_states"], load("sig_states")
    inp = make_chunkwise_inputs(case)
    fw = O.chunkwise_fw(inp["q"], inp["k"], inp["v"], inp["i"], inp["f"], chunk_size=L, siging=True)
    assert max_rel_err(fw["C_last"], gold["C_last"]) < TOL_FW
    assert max_rel_err(fw["n_last"], gold["n_last"]) < TOL_FW


def test_step_matches_reference():
    case, gold = CASES["step_small"], load("step_small")
    inp = make_step_inputs(case)
    c, n, m = inp["c"], inp["n"], inp["m"]
    for s in range(case["steps"]):
        h, (c, n, m) = O.recurrent_step(inp["q"][s], inp["k"][s], inp["v"][s], inp["i"][s], inp["f"][s], c, n, m)
        assert max_rel_err(h, gold["h"][s]) < TOL_FW
    for got, key in ((c, "c"), (n, "n"), (m, "m")):
        assert max_rel_err(got, gold[key]) < TOL_FW, key


@pytest.mark.parametrize("siging", [False, True])
def test_state_passing(siging):
    """Segment chaining through (C, n, m) reproduces the single pass
    (the reference's state-passing fixture: seed 42, (B,NH,S,DHQK,DHHV) = (2,4,256,16,32))."""
    case = dict(seed=42, B=2, NH=4, S=256, DHQK=16, DHHV=32, f_offset=3.0)
    inp = make_chunkwise_inputs(case)
    full = O.chunkwise_fw(inp["q"], inp["k"], inp["v"], inp["i"], inp["f"], chunk_size=32, siging=siging)
    c = n = m = None
    hs = []
    for s0 in range(0, 256, 64):
        sl = slice(s0, s0 + 64)
        seg = O.chunkwise_fw(inp["q"][:, :, sl], inp["k"][:, :, sl], inp["v"][:, :, sl], inp["i"][:, :, sl],
                             inp["f"][:, :, sl], c, n, m, chunk_size=32, siging=siging)
        c, n, m = seg["C_last"], seg["n_last"], seg["m_last"]
        hs.append(seg["H"])
    assert max_rel_err(np.concatenate(hs, 2), full["H"]) < 1e-10
    assert max_rel_err(c, full["C_last"]) < 1e-10
    assert max_rel_err(n, full["n_last"]) < 1e-10


def test_step_sequence_equals_chunkwise():
    """A loop of decode steps equals the chunkwise forward (the reference's recurrent-vs-parallel test)."""
    case = dict(seed=7, B=1, NH=2, S=64, DHQK=16, DHHV=32, f_offset=3.0)
    inp = make_chunkwise_inputs(case)
    fw = O.chunkwise_fw(inp["q"], inp["k"], inp["v"], inp["i"], inp["f"], chunk_size=16)
    c = np.zeros((1, 2, 16, 32)); n = np.zeros((1, 2, 16)); m = np.zeros((1, 2, 1))
    for t in range(64):
        h, (c, n, m) = O.recurrent_step(inp["q"][:, :, t], inp["k"][:, :, t], inp["v"][:, :, t],
                                        inp["i"][:, :, t, None], inp["f"][:, :, t, None], c, n, m)
        assert max_rel_err(h, fw["H"][:, :, t]) < 1e-6
    # states agree up to the common stabiliser scale
    assert max_rel_err(c * np.exp(m)[..., None], fw["C_last"] * np.exp(fw["m_last"])[..., None]) < 1e-8
