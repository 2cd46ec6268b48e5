"""Helpers for the GPU parity tests: run the CUDA path (through the Python shim over the C ABI)
and the numpy oracle on the same seeded inputs."""

from __future__ import annotations

import numpy as np
import torch

import mlstm_kernels_b200 as mk
from inputs import make_chunkwise_inputs
from oracle import mlstm_oracle as O

DEV = "cuda"
TDT = {"f32": torch.float32, "bf16": torch.bfloat16, "f16": torch.float16}


def to_dev(x, dtype, grad=False):
    t = torch.from_numpy(np.ascontiguousarray(x)).to(DEV).to(dtype)
    if grad:
        t.requires_grad_(True)
    return t


def rounded(x, dtype):
    """Inputs as the kernel sees them (rounded to the kernel dtype), back in float64 for the oracle."""
    return torch.from_numpy(np.ascontiguousarray(x)).to(dtype).to(torch.float64).numpy()


def npy(t):
    return None if t is None else t.detach().to(torch.float64).cpu().numpy()


def run_cuda_fwbw(inp, L, dtype=torch.float32, siging=False, normalize=True, impl="auto", eps=1e-6,
                  return_last_states=True):
    q, k, v, i, f = (to_dev(inp[n], dtype, True) for n in "qkvif")
    c0 = to_dev(inp["c0"], torch.float32, True) if "c0" in inp else None
    n0 = to_dev(inp["n0"], torch.float32) if "n0" in inp else None
    m0 = to_dev(inp["m0"], torch.float32) if "m0" in inp else None
    if siging:
        res = mk.mlstm_siging_chunkwise__b200_xl_chunk(q, k, v, i, f, c0, n0, None, return_last_states, eps,
                                                        normalize, chunk_size=L, impl=impl)
    else:
        res = mk.mlstm_chunkwise__b200_xl_chunk(q, k, v, i, f, c0, n0, m0, return_last_states, eps, chunk_size=L,
                                                impl=impl)
    if return_last_states:
        H, last = res
    else:
        H, last = res, None
    loss = (H.float() * to_dev(inp["dH"], torch.float32)).sum()
    if "dC_last" in inp and last is not None:
        loss = loss + (last[0] * to_dev(inp["dC_last"], torch.float32)).sum()
    loss.backward()
    out = dict(H=npy(H), dQ=npy(q.grad), dK=npy(k.grad), dV=npy(v.grad), dI=npy(i.grad), dF=npy(f.grad))
    if last is not None:
        out["C_last"], out["n_last"] = npy(last[0]), npy(last[1])
        if not siging:
            out["m_last"] = npy(last[2])
    if c0 is not None:
        out["dC_initial"] = npy(c0.grad)
    return out


def run_oracle_fwbw(inp, L, dtype=torch.float32, siging=False, normalize=True, eps=1e-6):
    r = {n: rounded(inp[n], dtype) for n in ("q", "k", "v", "i", "f", "dH")}
    fw, bw = O.chunkwise_fwbw(r["q"], r["k"], r["v"], r["i"], r["f"], r["dH"], c_initial=inp.get("c0"),
                              n_initial=inp.get("n0"), m_initial=None if siging else inp.get("m0"),
                              dC_last=inp.get("dC_last"), chunk_size=L, eps=eps, siging=siging, normalize=normalize)
    out = dict(H=fw["H"], C_last=fw["C_last"], n_last=fw["n_last"], m_last=fw["m_last"], **{
        n: bw[n] for n in ("dQ", "dK", "dV", "dI", "dF")})
    if bw["dC_initial"] is not None:
        out["dC_initial"] = bw["dC_initial"]
    return out


def case_inputs(seed, B, NH, S, DHQK, DHHV, f_offset=3.0, init=False, dC_last=False):
    return make_chunkwise_inputs(dict(seed=seed, B=B, NH=NH, S=S, DHQK=DHQK, DHHV=DHHV, f_offset=f_offset,
                                      init=init, dC_last=dC_last))
