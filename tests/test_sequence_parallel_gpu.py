"""Sequence-parallel prefill on GPUs.

* one GPU: the segment summary / state combine kernels and the scan-mode algebra are checked by
  emulating the ranks one after the other in a single process;
* two or more GPUs (skipped otherwise): real ranks under torchrun, NCCL point-to-point hand-off.
Tolerance: f32 states 1e-4 (bf16 inputs 2e-2 on H), against the single-pass result of the same kernels
and against the oracle."""

import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import mlstm_kernels_b200 as mk
from inputs import max_rel_err
from mlstm_kernels_b200 import _lib, sharding
from oracle import mlstm_oracle as O
from util_gpu import case_inputs, npy, rounded, to_dev

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("dtype,L,dims", [(torch.float32, 32, (16, 32)), (torch.bfloat16, 128, (128, 128)),
                                          (torch.bfloat16, 256, (256, 512))])
@pytest.mark.parametrize("siging", [False, True])
def test_scan_mode_emulated_on_one_gpu(dtype, L, dims, siging):
    DHQK, DHHV = dims
    P, S = 4, 4 * max(L, 128) * 2
    inp = case_inputs(31, 1, 2, S, DHQK, DHHV, f_offset=1.0)
    q, k, v, i, f = (to_dev(inp[n], dtype) for n in "qkvif")
    variant = _lib.SIG if siging else _lib.EXP
    fn = mk.mlstm_siging_chunkwise__b200_xl_chunk if siging else mk.mlstm_chunkwise__b200_xl_chunk
    h_full, last_full = fn(q, k, v, i, f, return_last_states=True, chunk_size=L)
    Lk = mk.kernel_chunk_size(q, v, L)
    seg = S // P
    state = (None, None, None)
    hs = []
    for r in range(P):
        sl = slice(r * seg, (r + 1) * seg)
        summ = sharding.segment_summary(k[:, :, sl], v[:, :, sl], i[:, :, sl], f[:, :, sl], chunk_size=Lk,
                                        variant=variant)
        h, _, _ = sharding._segment_forward_saved(q[:, :, sl], k[:, :, sl], v[:, :, sl], i[:, :, sl], f[:, :, sl],
                                                  state, chunk_size=Lk, eps=1e-6, variant=variant, impl="auto")
        state = sharding.state_combine(state, summ, variant=variant)
        hs.append(h)
    tol_h = 1e-5 if dtype == torch.float32 else 2e-2
    assert max_rel_err(npy(torch.cat(hs, 2)), npy(h_full)) < tol_h
    assert max_rel_err(npy(state[0]), npy(last_full[0])) < 1e-4
    assert max_rel_err(npy(state[1]), npy(last_full[1])) < 1e-4
    if not siging:
        assert max_rel_err(npy(state[2]), npy(last_full[2])) < 1e-5
    # and against the oracle on the same (rounded) inputs
    ref = O.chunkwise_fw(*(rounded(inp[n], dtype) for n in "qkvif"), chunk_size=Lk, siging=siging)
    assert max_rel_err(npy(torch.cat(hs, 2)), ref["H"]) < (1e-4 if dtype == torch.float32 else 2e-2)
    assert max_rel_err(npy(state[0]), ref["C_last"]) < (1e-4 if dtype == torch.float32 else 2e-2)


@pytest.mark.parametrize("dtype,L,dims", [(torch.float32, 32, (16, 32)), (torch.bfloat16, 128, (256, 256))])
@pytest.mark.parametrize("siging", [False, True])
def test_backward_chain_emulated_on_one_gpu(dtype, L, dims, siging):
    """The backward of the sequence-parallel mode, ranks emulated one after the other: segments are differentiated
    from the last to the first, each receiving the gradient of the state it handed over and the sum of
    (q . dq - k . dk) over all later tokens.  Compared with the single pass over the whole sequence."""
    DHQK, DHHV = dims
    P, S = 4, 4 * max(L, 128)
    inp = case_inputs(33, 1, 2, S, DHQK, DHHV, f_offset=1.0)
    q, k, v, i, f = (to_dev(inp[n], dtype) for n in "qkvif")
    dh = to_dev(inp["dH"], dtype)
    variant = _lib.SIG if siging else _lib.EXP
    fn = mk.mlstm_siging_chunkwise__b200_xl_chunk if siging else mk.mlstm_chunkwise__b200_xl_chunk
    leaves = [t.detach().clone().requires_grad_(True) for t in (q, k, v, i, f)]
    fn(*leaves, chunk_size=L).backward(dh)
    Lk = mk.kernel_chunk_size(q, v, L)
    seg = S // P
    state, saved = (None, None, None), []
    for r in range(P):
        sl = slice(r * seg, (r + 1) * seg)
        _, state, sv = sharding._segment_forward_saved(q[:, :, sl], k[:, :, sl], v[:, :, sl], i[:, :, sl], f[:, :, sl],
                                                       state, chunk_size=Lk, eps=1e-6, variant=variant, impl="auto")
        saved.append(sv)
    dc_last, tail, grads = None, None, [None] * P
    for r in reversed(range(P)):
        sl = slice(r * seg, (r + 1) * seg)
        qs, ks, vs, is_, fs = (t[:, :, sl].contiguous() for t in (q, k, v, i, f))
        dq, dk, dv, di, df, dc_last = sharding._segment_backward(qs, ks, vs, is_, fs, saved[r],
                                                                 dh[:, :, sl].contiguous(), dc_last, chunk_size=Lk,
                                                                 eps=1e-6, variant=variant, impl="auto")
        own = sharding._segment_gate_sum(qs, ks, fs, dq, dk, df)
        if tail is not None:
            df = df + torch.sigmoid(-fs.float()) * tail[..., None]
        tail = own if tail is None else own + tail
        grads[r] = (dq, dk, dv, di, df)
    tol = 1e-4 if dtype == torch.float32 else 2e-2
    for j, name in enumerate("qkvif"):
        got = torch.cat([g[j] for g in grads], 2)
        assert max_rel_err(npy(got), npy(leaves[j].grad)) < tol, name


@pytest.mark.parametrize("dtype,L,dims", [(torch.float32, 32, (16, 32)), (torch.bfloat16, 128, (256, 256)),
                                          (torch.float16, 128, (128, 256))])
@pytest.mark.parametrize("variant", [_lib.EXP, _lib.SIG, _lib.SIG_NONORM])
def test_backward_scan_emulated_on_one_gpu(dtype, L, dims, variant):
    """Scan form of the backward, ranks emulated in one process: (1) every segment's own state-gradient summary,
    (2) the boundary gradients by dC_left = a dC_right + dC_own, (3) every segment's full backward from its true
    dC_right, with the forget-gate tail <C_last, dC_right>.  Compared with the single pass over the whole sequence;
    the summary is also compared with the dC_initial that the full segment backward returns."""
    DHQK, DHHV = dims
    P, S = 4, 4 * max(L, 128)
    inp = case_inputs(35, 1, 2, S, DHQK, DHHV, f_offset=1.0)
    q, k, v, i, f = (to_dev(inp[n], dtype) for n in "qkvif")
    dh = to_dev(inp["dH"], dtype)
    siging = variant != _lib.EXP
    kw = dict(chunk_size=L)
    if siging:
        kw["normalize"] = variant == _lib.SIG
    fn = mk.mlstm_siging_chunkwise__b200_xl_chunk if siging else mk.mlstm_chunkwise__b200_xl_chunk
    leaves = [t.detach().clone().requires_grad_(True) for t in (q, k, v, i, f)]
    fn(*leaves, **kw).backward(dh)
    Lk = mk.kernel_chunk_size(q, v, L)
    seg = S // P
    opt = dict(chunk_size=Lk, eps=1e-6, variant=variant, impl="auto")
    cut = lambda t, r: t[:, :, r * seg:(r + 1) * seg].contiguous()  # noqa: E731
    state, saved, ends, decay = (None, None, None), [], [], []
    for r in range(P):
        g = torch.nn.functional.logsigmoid(cut(f, r).float()).sum(-1)
        m_in = torch.zeros_like(g) if state[2] is None else state[2].reshape(g.shape)
        _, state, sv = sharding._segment_forward_saved(*(cut(t, r) for t in (q, k, v, i, f)), state, **opt)
        saved.append(sv)
        ends.append(state[0])
        decay.append(torch.exp(g + m_in - state[2].reshape(g.shape)) if variant == _lib.EXP else torch.exp(g))
    own = [sharding.segment_dc_summary(cut(q, r), cut(dh, r), saved[r], **opt) for r in range(P)]
    dc_right = [None] * P
    for r in reversed(range(P - 1)):
        nxt = own[r + 1] if dc_right[r + 1] is None else own[r + 1] + decay[r + 1][..., None, None] * dc_right[r + 1]
        dc_right[r] = nxt
    grads = []
    for r in range(P):
        dq, dk, dv, di, df, dc0 = sharding._segment_backward(*(cut(t, r) for t in (q, k, v, i, f)), saved[r], cut(dh, r),
                                                             dc_right[r], **opt)
        if dc_right[r] is not None:
            tail = (ends[r] * dc_right[r]).sum(dim=(-1, -2))
            df = df + torch.sigmoid(-cut(f, r).float()) * tail[..., None]
        else:   # last segment: its own summary IS the gradient of the state it received
            assert max_rel_err(npy(own[r]), npy(dc0)) < 1e-5
        grads.append((dq, dk, dv, di, df))
    tol = 1e-4 if dtype == torch.float32 else 2e-2
    for j, name in enumerate("qkvif"):
        got = torch.cat([g_[j] for g_ in grads], 2)
        assert max_rel_err(npy(got), npy(leaves[j].grad)) < tol, name


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs at least two GPUs")
@pytest.mark.parametrize("mode", ["gather", "scan", "chain"])
def test_sequence_parallel_torchrun(tmp_path, mode):
    n = min(torch.cuda.device_count(), 4)
    script = os.path.join(os.path.dirname(os.path.abspath(__file__)), "run_sequence_parallel.py")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={n}",
                        "--master-addr", "127.0.0.1", "--master-port", "29613", script, "--mode", mode,
                        "--out", str(tmp_path)], capture_output=True, text=True, env=env, timeout=600)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-4000:]
    res = dict(np.load(tmp_path / "result.npz"))
    assert res["err_h"] < 2e-2 and res["err_c"] < 1e-4 and res["err_n"] < 1e-4 and res["err_m"] < 1e-5
    for n in "qkvif":   # backward chain against the single-GPU backward of the whole sequence
        assert res["err_d" + n] < 2e-2, n
