"""Outputs of the B200 kernels next to the reference's own Triton kernels on the same GPU and the same seeded inputs.

Needs the reference package to be importable (e.g. `pip install --no-deps --target baseline/_ref <reference
checkout>`); skipped otherwise, and a kernel the machine's Triton cannot compile is reported as a skip with the
compiler's message rather than a failure of this library.

Tolerances: the reference's own ones for its Triton kernels (tests/torch/chunkwise/test_chunkwise_triton_xl_chunk.py:
forward atol 2e-2 / rtol 5e-2 element-wise; its backward tolerances, atol 4.2 / rtol 0.5, are too loose to mean
anything, so the gradients use this suite's measure instead: max |x - ref| / max |ref| < 2e-2 in f32 and < 3e-2 in
bf16, where both sides carry their own bf16 rounding).  Known, documented differences that stay inside these
bounds: the Triton kernels clamp the intra-chunk max state at -10 and store the per-token denominator in the input
dtype (mlstm_kernels/torch/chunkwise/triton_xl_chunk/fw_parallel.py:80-81,130).
"""

import os
import sys

import numpy as np
import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
_ref = os.path.join(ROOT, "baseline", "_ref")
if os.path.isdir(_ref) and _ref not in sys.path:
    sys.path.insert(0, _ref)
pytest.importorskip("mlstm_kernels")
pytest.importorskip("triton")

import mlstm_kernels_b200 as mk  # noqa: E402
from inputs import elementwise_ok_fraction, max_rel_err  # noqa: E402
from util_gpu import case_inputs, npy, to_dev  # noqa: E402

pytestmark = pytest.mark.gpu


def _run(fn, inp, dtype, L, **kw):
    leaves = [to_dev(inp[n], dtype, True) for n in "qkvif"]
    try:
        h, last = fn(*leaves, return_last_states=True, chunk_size=L, **kw)
        h.backward(to_dev(inp["dH"], dtype))
    except Exception as e:  # noqa: BLE001  (Triton compile / API errors of the reference on this machine)
        if fn.__module__.startswith("mlstm_kernels."):
            pytest.skip(f"reference Triton kernel unavailable on this machine: {type(e).__name__}: {str(e)[:200]}")
        raise
    return npy(h), [npy(t) for t in last], [npy(t.grad) for t in leaves]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("shape", [(2, 2, 512, 128, 128, 64), (1, 4, 1024, 256, 256, 128)])
def test_mlstmexp_vs_triton_xl_chunk(shape, dtype):
    from mlstm_kernels.torch.chunkwise.triton_xl_chunk import mlstm_chunkwise__xl_chunk
    B, NH, S, DHQK, DHHV, L = shape
    inp = case_inputs(61, B, NH, S, DHQK, DHHV)
    h_r, last_r, g_r = _run(mlstm_chunkwise__xl_chunk, inp, dtype, L)
    h_b, last_b, g_b = _run(mk.mlstm_chunkwise__b200_xl_chunk, inp, dtype, L)
    tol = 2e-2 if dtype == torch.float32 else 3e-2
    print(f"\nmLSTMexp vs Triton {shape} {dtype}: H max|diff| {np.abs(h_b - h_r).max():.3e}, max-normalised "
          f"{max_rel_err(h_b, h_r):.3e}; grads " + " ".join(f"{max_rel_err(a, b):.2e}" for a, b in zip(g_b, g_r)))
    if dtype == torch.float32:
        assert np.allclose(h_b, h_r, atol=2e-2, rtol=5e-2)      # the reference's own forward tolerance
    else:   # two bf16 pipelines: each output carries its own rounding (one bf16 ulp of |h| ~ 4 is 3e-2)
        assert elementwise_ok_fraction(h_b, h_r, 5e-2, 3e-2) >= 0.999
    assert max_rel_err(h_b, h_r) < tol
    for name, a, b in zip(("dQ", "dK", "dV", "dI", "dF"), g_b, g_r):
        # in bf16 the Triton path forms deltaF from its ROUNDED deltaQ, deltaK outputs
        # (mlstm_kernels/torch/chunkwise/triton_xl_chunk/chunkwise_gates.py:68-95): q.dq - k.dk nearly cancel, so
        # that rounding dominates the difference; this library sums the f32 accumulators
        assert max_rel_err(a, b) < (6e-2 if (name == "dF" and dtype == torch.bfloat16) else tol), name
    # (C, n, m) triples agree up to the common stabiliser scale exp(m)
    tol_s = 1e-3 if dtype == torch.float32 else 2e-2
    sc_b, sc_r = np.exp(last_b[2])[..., None], np.exp(last_r[2])[..., None]
    assert max_rel_err(last_b[0] * sc_b, last_r[0] * sc_r) < tol_s
    assert max_rel_err(last_b[1] * sc_b[..., 0], last_r[1] * sc_r[..., 0]) < tol_s


@pytest.mark.parametrize("normalize", [True, False])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_mlstmsig_vs_triton_xl_chunk_siging(dtype, normalize):
    from mlstm_kernels.torch.chunkwise.triton_xl_chunk_siging import mlstm_siging_chunkwise__xl_chunk
    B, NH, S, DHQK, DHHV, L = 1, 4, 1024, 256, 256, 128
    inp = case_inputs(62, B, NH, S, DHQK, DHHV)
    h_r, last_r, g_r = _run(mlstm_siging_chunkwise__xl_chunk, inp, dtype, L, normalize=normalize)
    h_b, last_b, g_b = _run(mk.mlstm_siging_chunkwise__b200_xl_chunk, inp, dtype, L, normalize=normalize)
    tol = 2e-2 if dtype == torch.float32 else 3e-2
    print(f"\nmLSTMsig normalize={normalize} vs Triton {dtype}: H max|diff| {np.abs(h_b - h_r).max():.3e}, max-normalised "
          f"{max_rel_err(h_b, h_r):.3e}; grads " + " ".join(f"{max_rel_err(a, b):.2e}" for a, b in zip(g_b, g_r)))
    assert np.allclose(h_b, h_r, atol=2e-2 * max(1.0, np.abs(h_r).max()), rtol=5e-2)
    assert max_rel_err(h_b, h_r) < tol
    for name, a, b in zip(("dQ", "dK", "dV", "dI", "dF"), g_b, g_r):
        assert max_rel_err(a, b) < (6e-2 if (name == "dF" and dtype == torch.bfloat16) else tol), name
    assert max_rel_err(last_b[0], last_r[0]) < (1e-3 if dtype == torch.float32 else 2e-2)
    if normalize:
        assert max_rel_err(last_b[1], last_r[1]) < (1e-3 if dtype == torch.float32 else 2e-2)


@pytest.mark.parametrize("B", [1, 8])
def test_step_vs_triton_step(B):
    from mlstm_kernels.torch.recurrent.triton_step import mlstm_recurrent_step__triton
    NH, DHQK, DHHV = 8, 256, 512
    g = torch.Generator(device="cuda").manual_seed(63)
    c = torch.randn(B, NH, DHQK, DHHV, device="cuda", generator=g) * 0.1
    n = torch.randn(B, NH, DHQK, device="cuda", generator=g).abs()
    m = torch.randn(B, NH, 1, device="cuda", generator=g)
    q, k = (torch.randn(B, NH, DHQK, device="cuda", generator=g).bfloat16() for _ in range(2))
    v = torch.randn(B, NH, DHHV, device="cuda", generator=g).bfloat16()
    i = torch.randn(B, NH, 1, device="cuda", generator=g).bfloat16()
    f = (3 + torch.randn(B, NH, 1, device="cuda", generator=g)).bfloat16()
    try:
        h_r, (c_r, n_r, m_r) = mlstm_recurrent_step__triton(q, k, v, i, f, c, n, m)
    except Exception as e:  # noqa: BLE001
        pytest.skip(f"reference Triton step kernel unavailable on this machine: {type(e).__name__}: {str(e)[:200]}")
    h_b, (c_b, n_b, m_b) = mk.mlstm_recurrent_step__b200(q, k, v, i, f, c, n, m)
    # The Triton kernel rounds the gate activations exp(lf + m - m'), exp(i - m') and C' to the input dtype (bf16)
    # before it uses them (mlstm_kernels/triton/recurrent/fw_step_fused.py:101-105,185), so its new state carries
    # one bf16 rounding (2^-8 relative) that the f32 arithmetic of this library does not have.
    assert max_rel_err(npy(h_b), npy(h_r)) < 3e-2
    assert max_rel_err(npy(c_b), npy(c_r)) < 1e-2
    assert max_rel_err(npy(n_b), npy(n_r)) < 1e-2
    assert max_rel_err(npy(m_b), npy(m_r)) < 1e-6
