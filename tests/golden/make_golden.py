"""Generate the golden vectors in this folder by running the reference's own PyTorch code on CPU.

Usage (only where the reference source tree is available):

    python tests/golden/make_golden.py /path/to/mlstm_kernels_checkout

Inputs are drawn with numpy's PCG64 generator (platform independent) by `tests/inputs.py`,
so the tests can regenerate them bit-for-bit; only the reference OUTPUTS are stored
(float32, npz-compressed; the largest case is stored on a strided sub-grid).
"""

from __future__ import annotations

import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))
from inputs import CASES, make_chunkwise_inputs, make_step_inputs, subsample  # noqa: E402


def t(x, grad=False):
    y = torch.from_numpy(np.ascontiguousarray(x)).clone()
    if grad:
        y.requires_grad_(True)
    return y


def run_exp_chunkwise(case):
    from mlstm_kernels.torch.chunkwise.native.fw import mlstm_chunkwise_fw
    from mlstm_kernels.torch.chunkwise.native.fwbw import mlstm_chunkwise__native_custbw

    inp = make_chunkwise_inputs(case)
    q, k, v, i, f = (t(inp[n], True) for n in "qkvif")
    c0 = t(inp["c0"], True) if "c0" in inp else None
    n0 = t(inp["n0"]) if "n0" in inp else None
    m0 = t(inp["m0"]) if "m0" in inp else None
    L = case["L"]
    with torch.no_grad():
        H, n_out, m_out, last, allst = mlstm_chunkwise_fw(
            q, k, v, i, f, c0, n0, m0, return_last_states=True, return_all_states=True, chunk_size=L, eps=1e-6)
    out = dict(H=H, n_out=n_out, m_out=m_out, C_last=last[0], n_last=last[1], m_last=last[2])
    B, NH, S, DHQK = q.shape
    NC = S // L
    out["C_states"] = allst[0].reshape(B, NH, NC + 1, DHQK, -1)
    out["n_states"] = allst[1].reshape(B, NH, NC + 1, DHQK)
    out["m_states"] = allst[2]
    # custom backward (drops the denominator gradient)
    H2, last2 = mlstm_chunkwise__native_custbw(q, k, v, i, f, c0, n0, m0, return_last_states=True, chunk_size=L, eps=1e-6)
    loss = (H2 * t(inp["dH"])).sum()
    if "dC_last" in inp:
        loss = loss + (last2[0] * t(inp["dC_last"])).sum()
    loss.backward()
    out.update(dQ=q.grad, dK=k.grad, dV=v.grad, dI=i.grad, dF=f.grad)
    if c0 is not None:
        out["dC_initial"] = c0.grad
    return {n: x.detach().numpy().astype(np.float32) for n, x in out.items()}


def run_exp_parallel(case):
    from mlstm_kernels.torch.parallel.native_stablef.fwbw import mlstm_parallel__native_stablef_custbw

    inp = make_chunkwise_inputs(case)
    q, k, v, i, f = (t(inp[n], True) for n in "qkvif")
    H = mlstm_parallel__native_stablef_custbw(q, k, v, i, f, eps=1e-6)
    (H * t(inp["dH"])).sum().backward()
    out = dict(H=H, dQ=q.grad, dK=k.grad, dV=v.grad, dI=i.grad, dF=f.grad)
    return {n: x.detach().numpy().astype(np.float32) for n, x in out.items()}


def run_sig_parallel(case):
    from mlstm_kernels.torch.parallel.native_siging.fwbw import mlstm_siging_parallel__native_custbw

    inp = make_chunkwise_inputs(case)
    q, k, v, i, f = (t(inp[n], True) for n in "qkvif")
    H = mlstm_siging_parallel__native_custbw(q, k, v, i, f, eps=1e-6, stable_fgate=True, normalize=case["normalize"])
    (H * t(inp["dH"])).sum().backward()
    out = dict(H=H, dQ=q.grad, dK=k.grad, dV=v.grad, dI=i.grad, dF=f.grad)
    return {n: x.detach().numpy().astype(np.float32) for n, x in out.items()}


def run_sig_states(case):
    """Final mLSTMsig state (C_last, n_last) out of the reference's quadratic implementation, which returns H only.
    DHQK probe tokens are appended to the sequence: probe d has q = e_d / qk_scale, k = 0, v = 0 and a forget logit of
    +40 (logsigmoid = 0 in f32), so it adds nothing to the state, nothing decays, and its un-normalised output row is
    H_probe[d, :] = sum_j exp(sum_{t>j} logsigmoid f_t + logsigmoid i_j) k_j[d] v_j = C_last[d, :].  A second run with
    every v set to ones gives n_last[d] in every output column."""
    from mlstm_kernels.torch.parallel.native_siging.fwbw import mlstm_siging_parallel__native_custbw

    inp = make_chunkwise_inputs(case)
    B, NH, S, DHQK = inp["q"].shape
    DHHV = inp["v"].shape[-1]
    probe_q = np.broadcast_to((np.eye(DHQK) * np.sqrt(DHQK)).astype(np.float32), (B, NH, DHQK, DHQK))
    q = np.concatenate([inp["q"], probe_q], 2)
    k = np.concatenate([inp["k"], np.zeros((B, NH, DHQK, DHQK), np.float32)], 2)
    v = np.concatenate([inp["v"], np.zeros((B, NH, DHQK, DHHV), np.float32)], 2)
    i = np.concatenate([inp["i"], np.zeros((B, NH, DHQK), np.float32)], 2)
    f = np.concatenate([inp["f"], np.full((B, NH, DHQK), 40.0, np.float32)], 2)
    with torch.no_grad():
        H = mlstm_siging_parallel__native_custbw(t(q), t(k), t(v), t(i), t(f), eps=1e-6, stable_fgate=True,
                                                 normalize=False)
        Hn = mlstm_siging_parallel__native_custbw(t(q), t(k), t(np.ones_like(v)), t(i), t(f), eps=1e-6,
                                                  stable_fgate=True, normalize=False)
    out = dict(C_last=H[:, :, S:], n_last=Hn[:, :, S:, 0])
    return {n_: x.detach().numpy().astype(np.float32) for n_, x in out.items()}


def run_step(case):
    from mlstm_kernels.torch.recurrent.native_step import mlstm_recurrent_step__native

    inp = make_step_inputs(case)
    c, n, m = t(inp["c"]), t(inp["n"]), t(inp["m"])
    hs = []
    for s in range(case["steps"]):
        h, (c, n, m) = mlstm_recurrent_step__native(
            t(inp["q"][s]), t(inp["k"][s]), t(inp["v"][s]), t(inp["i"][s]), t(inp["f"][s]), c, n, m, eps=1e-6)
        hs.append(h)
    out = dict(h=torch.stack(hs), c=c, n=n, m=m)
    return {n_: x.detach().numpy().astype(np.float32) for n_, x in out.items()}


RUNNERS = dict(exp_chunkwise=run_exp_chunkwise, exp_parallel=run_exp_parallel, sig_parallel=run_sig_parallel,
               sig_states=run_sig_states, step=run_step)


def main():
    ref_root = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("MLSTM_REFERENCE_ROOT", "")
    if not ref_root or not os.path.isdir(os.path.join(ref_root, "mlstm_kernels")):
        raise SystemExit("pass the path of a checkout of the reference (the folder that holds mlstm_kernels/)")
    sys.path.insert(0, ref_root)
    torch.set_num_threads(os.cpu_count() or 1)
    for name, case in CASES.items():
        out = RUNNERS[case["kind"]](case)
        out = {n: subsample(x, case.get("stride", 1)) for n, x in out.items()}
        path = os.path.join(HERE, f"{name}.npz")
        np.savez_compressed(path, **out)
        print(f"{name}: {os.path.getsize(path) / 1e6:.2f} MB  " + " ".join(f"{n}{tuple(x.shape)}" for n, x in out.items()))


if __name__ == "__main__":
    main()
