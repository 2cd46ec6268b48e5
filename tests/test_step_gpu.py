"""GPU parity tests of the recurrent decode kernels vs the oracle and the reference golden vectors.
Tolerances: f32 1e-5 on h and states; bf16 inputs 2e-2 on h, f32 states 1e-4 (oracle fed bf16-rounded inputs)."""

import os

import numpy as np
import pytest
import torch

import mlstm_kernels_b200 as mk
from inputs import CASES, make_step_inputs, max_rel_err
from oracle import mlstm_oracle as O
from util_gpu import case_inputs, npy, rounded, to_dev

pytestmark = pytest.mark.gpu
GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def test_step_f32_vs_reference_golden():
    case = CASES["step_small"]
    gold = dict(np.load(os.path.join(GOLD, "step_small.npz")))
    inp = make_step_inputs(case)
    c, n, m = (to_dev(inp[x], torch.float32) for x in "cnm")
    for s in range(case["steps"]):
        q, k, v, i, f = (to_dev(inp[x][s], torch.float32) for x in "qkvif")
        c_old = c.clone()
        h, (c2, n2, m2) = mk.mlstm_recurrent_step__b200(q, k, v, i, f, c, n, m)
        assert torch.equal(c, c_old), "old state must stay untouched"
        c, n, m = c2, n2, m2
        assert max_rel_err(npy(h), gold["h"][s]) < 1e-5
    assert max_rel_err(npy(c), gold["c"]) < 1e-5
    assert max_rel_err(npy(n), gold["n"]) < 1e-5
    assert max_rel_err(npy(m), gold["m"]) < 1e-5


@pytest.mark.parametrize("B,NH,DHQK,DHHV", [(1, 8, 256, 512), (8, 8, 256, 512), (3, 2, 48, 96), (2, 4, 64, 128)])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32, torch.float16])
def test_step_vs_oracle(B, NH, DHQK, DHHV, dtype):
    inp = make_step_inputs(dict(seed=9, B=B, NH=NH, DHQK=DHQK, DHHV=DHHV, steps=3))
    c, n, m = (to_dev(inp[x], torch.float32) for x in "cnm")
    co, no, mo = inp["c"], inp["n"], inp["m"]
    for s in range(3):
        q, k, v, i, f = (to_dev(inp[x][s], dtype) for x in "qkvif")
        h, (c, n, m) = mk.mlstm_recurrent_step__b200(q, k, v, i, f, c, n, m)
        ho, (co, no, mo) = O.recurrent_step(*(rounded(inp[x][s], dtype) for x in "qkvif"), co, no, mo)
        assert max_rel_err(npy(h), ho) < (1e-5 if dtype == torch.float32 else 2e-2)
    assert max_rel_err(npy(c), co) < 1e-4
    assert max_rel_err(npy(n), no) < 1e-4
    assert max_rel_err(npy(m), mo) < 1e-4


def test_step_bf16_tokens_with_f32_gates():
    """bf16 q, k, v next to f32 gate pre-activations (the usual xLSTM set-up): the gates reach the kernel unrounded
    and are widened to f32 as the reference does (mlstm_kernels/triton/recurrent/fw_step_fused.py:88-94).  Large gate
    values make the difference visible: rounding i ~ 8 to bf16 moves exp(i - m) by up to 3 %."""
    inp = make_step_inputs(dict(seed=12, B=2, NH=4, DHQK=64, DHHV=128, steps=2))
    inp["i"] = (inp["i"] * 4 + 6).astype(np.float32)
    c, n, m = (to_dev(inp[x], torch.float32) for x in "cnm")
    co, no, mo = inp["c"], inp["n"], inp["m"]
    for s in range(2):
        q, k, v = (to_dev(inp[x][s], torch.bfloat16) for x in "qkv")
        i, f = (to_dev(inp[x][s], torch.float32) for x in "if")
        h, (c, n, m) = mk.mlstm_recurrent_step__b200(q, k, v, i, f, c, n, m)
        ho, (co, no, mo) = O.recurrent_step(*(rounded(inp[x][s], torch.bfloat16) for x in "qkv"), inp["i"][s], inp["f"][s],
                                            co, no, mo)
        assert max_rel_err(npy(h), ho) < 2e-2
    # states carry no bf16 rounding of the gates: f32 accuracy
    assert max_rel_err(npy(c), co) < 1e-4
    assert max_rel_err(npy(n), no) < 1e-4
    assert max_rel_err(npy(m), mo) < 1e-5
    # the sequence kernel takes the gates the same way
    T = 8
    cw = case_inputs(13, 1, 2, T, 64, 128)
    q, k, v = (to_dev(cw[x], torch.bfloat16) for x in "qkv")
    gi, gf = to_dev(cw["i"] * 4 + 6, torch.float32), to_dev(cw["f"], torch.float32)
    h_seq, (c_s, _, m_s) = mk.mlstm_recurrent_sequence__b200(q, k, v, gi, gf, return_last_states=True)
    c = torch.zeros(1, 2, 64, 128, device="cuda"); n = torch.zeros(1, 2, 64, device="cuda"); m = torch.zeros(1, 2, 1, device="cuda")
    for t in range(T):
        h, (c, n, m) = mk.mlstm_recurrent_step__b200(q[:, :, t], k[:, :, t], v[:, :, t], gi[:, :, t, None],
                                                     gf[:, :, t, None], c, n, m)
    assert max_rel_err(npy(c_s), npy(c)) < 1e-5
    assert max_rel_err(npy(m_s), npy(m)) < 1e-6
    assert max_rel_err(npy(h_seq[:, :, -1]), npy(h)) < 1e-2


def test_step_bf16_state_and_out_buffers():
    inp = make_step_inputs(dict(seed=10, B=2, NH=2, DHQK=64, DHHV=128, steps=1))
    q, k, v, i, f = (to_dev(inp[x][0], torch.bfloat16) for x in "qkvif")
    c, n, m = (to_dev(inp[x], torch.bfloat16) for x in "cnm")
    h, (c2, n2, m2) = mk.mlstm_recurrent_step__b200(q, k, v, i, f, c, n, m, dtype_state=torch.bfloat16)
    assert c2.dtype == torch.bfloat16 and h.dtype == torch.bfloat16
    ho, (co, _, _) = O.recurrent_step(*(rounded(inp[x][0], torch.bfloat16) for x in "qkvif"),
                                      *(rounded(inp[x], torch.bfloat16) for x in "cnm"))
    assert max_rel_err(npy(h), ho) < 2e-2
    assert max_rel_err(npy(c2), co) < 1e-2
    # caller-provided output buffers; C may be updated in place
    cf = c.float()
    nb, mb = torch.empty_like(n, dtype=torch.float32), torch.empty_like(m, dtype=torch.float32)
    h3, (c3, n3, m3) = mk.mlstm_recurrent_step__b200_fw(cf, n.float(), m.float(), q, k, v, i, f, matC_new=cf,
                                                        vecN_new=nb, scaM_new=mb)
    assert c3.data_ptr() == cf.data_ptr()
    assert max_rel_err(npy(h3), ho) < 2e-2
    # decode loop that owns its buffers: validation off, same result
    cf2, nf2, mf2 = c.float(), n.float(), m.float()
    co, no, mo, hf = torch.empty_like(cf2), torch.empty_like(nf2), torch.empty_like(mf2), torch.empty_like(v)
    h5, (c5, _, _) = mk.mlstm_recurrent_step__b200_fw(cf2, nf2, mf2, q, k, v, i, f, matC_new=co, vecN_new=no,
                                                      scaM_new=mo, vecH_out=hf, validate=False)
    h6, (c6, _, _) = mk.mlstm_recurrent_step__b200_fw(cf2, nf2, mf2, q, k, v, i, f)
    assert torch.equal(h5, h6) and torch.equal(c5, c6)
    # caller-owned h
    hb = torch.empty_like(v)
    h4, _ = mk.mlstm_recurrent_step__b200_fw(c.float(), n.float(), m.float(), q, k, v, i, f, vecH_out=hb)
    assert h4.data_ptr() == hb.data_ptr()
    assert max_rel_err(npy(h4), ho) < 2e-2


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_sequence_kernel_equals_step_loop_and_chunkwise(dtype):
    inp = case_inputs(21, 2, 2, 32, 64, 128)
    q, k, v, i, f = (to_dev(inp[x], dtype) for x in "qkvif")
    h_seq, (c_s, n_s, m_s) = mk.mlstm_recurrent_sequence__b200(q, k, v, i, f, return_last_states=True)
    c = torch.zeros(2, 2, 64, 128, device="cuda"); n = torch.zeros(2, 2, 64, device="cuda")
    m = torch.zeros(2, 2, 1, device="cuda")
    hs = []
    for t in range(32):
        h, (c, n, m) = mk.mlstm_recurrent_step__b200(q[:, :, t], k[:, :, t], v[:, :, t], i[:, :, t, None],
                                                     f[:, :, t, None], c, n, m)
        hs.append(h)
    tol = 1e-5 if dtype == torch.float32 else 1e-2
    assert max_rel_err(npy(h_seq), npy(torch.stack(hs, 2))) < tol
    assert max_rel_err(npy(c_s), npy(c)) < 1e-5
    h_cw = mk.mlstm_chunkwise__b200_xl_chunk(q, k, v, i, f, chunk_size=16)
    assert max_rel_err(npy(h_seq), npy(h_cw)) < (1e-4 if dtype == torch.float32 else 2e-2)


def test_step_full_size_decay_property():
    """Size-independent check at the full decode geometry (B=64, NH=8, 256/512): with k = 0 the step
    must scale C by exp(logsigmoid(f) + m - m') exactly and leave it otherwise unchanged."""
    B, NH, DHQK, DHHV = 64, 8, 256, 512
    g = torch.Generator(device="cuda").manual_seed(0)
    c = torch.randn(B, NH, DHQK, DHHV, device="cuda", generator=g) * 0.1
    n = torch.randn(B, NH, DHQK, device="cuda", generator=g).abs()
    m = torch.randn(B, NH, 1, device="cuda", generator=g)
    q = torch.randn(B, NH, DHQK, device="cuda", generator=g).bfloat16()
    k = torch.zeros_like(q)
    v = torch.randn(B, NH, DHHV, device="cuda", generator=g).bfloat16()
    i = torch.randn(B, NH, 1, device="cuda", generator=g).bfloat16()
    f = (3 + torch.randn(B, NH, 1, device="cuda", generator=g)).bfloat16()
    h, (c2, n2, m2) = mk.mlstm_recurrent_step__b200(q, k, v, i, f, c, n, m)
    lf = torch.nn.functional.logsigmoid(f.float())
    m_new = torch.maximum(lf + m, i.float())
    scale = torch.exp(lf + m - m_new)
    assert torch.allclose(m2, m_new, rtol=1e-6, atol=1e-6)
    assert torch.allclose(c2, c * scale[..., None], rtol=1e-5, atol=1e-7)
    assert torch.allclose(n2, n * scale, rtol=1e-5, atol=1e-7)


def test_more_than_65535_batch_heads():
    """Batch x heads beyond the 65535 limit of a grid's second dimension (all grids are one-dimensional): decode step,
    multi-token sequence kernel and the chunkwise forward + backward on both kernel families, tiny head dims so that
    70 000 units stay small.  A unit computed inside the big launch equals the same unit computed alone, bit for bit,
    and a sample of units matches the oracle."""
    B, NH, D, S = 8750, 8, 8, 16          # 70 000 units
    g = torch.Generator(device="cuda").manual_seed(3)
    rnd = lambda *s: torch.randn(*s, device="cuda", generator=g)  # noqa: E731
    c, n, m = rnd(B, NH, D, D) * 0.1, rnd(B, NH, D).abs(), rnd(B, NH, 1)
    q, k, v = rnd(B, NH, S, D).bfloat16(), rnd(B, NH, S, D).bfloat16(), rnd(B, NH, S, D).bfloat16()
    i, f = rnd(B, NH, S).bfloat16(), (3 + rnd(B, NH, S)).bfloat16()
    pick = [0, 8191, 8749]                # first, one past the 65535th unit's batch row, last
    # decode step and sequence kernel
    h, st = mk.mlstm_recurrent_step__b200(q[:, :, 0], k[:, :, 0], v[:, :, 0], i[:, :, :1], f[:, :, :1], c, n, m)
    hs, sts = mk.mlstm_recurrent_sequence__b200(q, k, v, i, f, c, n, m, return_last_states=True)
    for b in pick:
        sl = slice(b, b + 1)
        h1, st1 = mk.mlstm_recurrent_step__b200(q[sl, :, 0], k[sl, :, 0], v[sl, :, 0], i[sl, :, :1], f[sl, :, :1],
                                                c[sl], n[sl], m[sl])
        assert torch.equal(h[sl], h1) and all(torch.equal(a[sl], b_) for a, b_ in zip(st, st1))
        hs1, sts1 = mk.mlstm_recurrent_sequence__b200(q[sl], k[sl], v[sl], i[sl], f[sl], c[sl], n[sl], m[sl],
                                                      return_last_states=True)
        assert torch.equal(hs[sl], hs1) and all(torch.equal(a[sl], b_) for a, b_ in zip(sts, sts1))
    # chunkwise: tensor-core kernels (bf16) and portable kernels (f32)
    dh = rnd(B, NH, S, D)
    for dtype in (torch.bfloat16, torch.float32):
        leaves = [t.to(dtype).detach().requires_grad_(True) for t in (q, k, v, i, f)]
        H = mk.mlstm_chunkwise__b200_xl_chunk(*leaves, chunk_size=16)
        H.backward(dh.to(dtype))
        for b in pick:
            sl = slice(b, b + 1)
            one = [t[sl].detach().clone().requires_grad_(True) for t in leaves]
            H1 = mk.mlstm_chunkwise__b200_xl_chunk(*one, chunk_size=16)
            H1.backward(dh[sl].to(dtype))
            assert torch.equal(H[sl], H1)
            for a, b_ in zip(leaves, one):
                assert torch.equal(a.grad[sl], b_.grad)
        ref = O.chunkwise_fw(*(npy(t[-1:]) for t in leaves), chunk_size=16)
        assert max_rel_err(npy(H[-1:]), ref["H"]) < (2e-2 if dtype == torch.bfloat16 else 1e-4)
