"""The public functions under torch.compile (fullgraph: no graph break allowed).  While a trace is taken they go
through the custom operators of mlstm_kernels_b200/_ops.py; the compiled results must equal the eager ones bit for
bit (same kernels, same inputs).  The reference's callers compile their models
(mlstm_kernels/utils/benchmark/benchmarks/interface.py:94-95)."""

import pytest
import torch

import mlstm_kernels_b200 as mk
from util_gpu import case_inputs, to_dev

pytestmark = pytest.mark.gpu


def _leaves(inp, dtype):
    return [to_dev(inp[n], dtype).requires_grad_(True) for n in "qkvif"]


@pytest.mark.parametrize("variant", ["exp", "sig"])
@pytest.mark.parametrize("recompute", [True, False])
def test_chunkwise_forward_backward_compiles_without_graph_break(variant, recompute):
    inp = case_inputs(61, 2, 2, 300, 128, 256, init=True)
    dh = to_dev(inp["dH"], torch.bfloat16)
    c0, n0, m0 = (to_dev(inp[n], torch.float32) for n in ("c0", "n0", "m0"))
    fn = mk.mlstm_chunkwise__b200_xl_chunk if variant == "exp" else mk.mlstm_siging_chunkwise__b200_xl_chunk

    def loss(q, k, v, i, f, c0):
        h, last = fn(q, k, v, i, f, c0, n0, m0 if variant == "exp" else None, return_last_states=True,
                     chunk_size=128, recompute_states_in_bw=recompute)
        return (h.float() * dh.float()).sum() + last[0].sum(), h, last

    def run(fun):
        leaves = _leaves(inp, torch.bfloat16)
        c = c0.clone().requires_grad_(True)
        val, h, last = fun(*leaves, c)
        val.backward()
        return [h.detach(), last[0].detach(), last[1].detach()] + [t.grad for t in leaves] + [c.grad]

    eager = run(loss)
    compiled = run(torch.compile(loss, fullgraph=True))
    for a, b in zip(eager, compiled):
        assert torch.equal(a, b)


def test_chunkwise_under_autocast_compiles():
    """Inside an autocast region the inputs are cast to autocast_kernel_dtype (f32 inputs, bf16 kernel)."""
    inp = case_inputs(62, 1, 2, 256, 128, 128)

    def f(q, k, v, i, f_):
        with torch.autocast("cuda", dtype=torch.bfloat16):
            return mk.mlstm_chunkwise__b200_xl_chunk(q, k, v, i, f_, chunk_size=128,
                                                     autocast_kernel_dtype=torch.bfloat16)
    args = [to_dev(inp[n], torch.float32) for n in "qkvif"]
    eager = f(*args)
    compiled = torch.compile(f, fullgraph=True)(*args)
    assert eager.dtype == torch.bfloat16 and torch.equal(eager, compiled)


def test_decode_step_and_sequence_compile():
    g = torch.Generator(device="cuda").manual_seed(7)
    B, NH, DHQK, DHHV, T = 2, 4, 128, 256, 6
    rnd = lambda *s: torch.randn(*s, device="cuda", generator=g)  # noqa: E731
    c, n, m = rnd(B, NH, DHQK, DHHV) * 0.1, rnd(B, NH, DHQK).abs(), rnd(B, NH, 1)
    q, k, v = rnd(B, NH, T, DHQK).bfloat16(), rnd(B, NH, T, DHQK).bfloat16(), rnd(B, NH, T, DHHV).bfloat16()
    i, f = rnd(B, NH, T).bfloat16(), (3 + rnd(B, NH, T)).bfloat16()

    def loop(q, k, v, i, f, c, n, m):
        hs = []
        for t in range(T):
            h, (c, n, m) = mk.mlstm_recurrent_step__b200(q[:, :, t], k[:, :, t], v[:, :, t], i[:, :, t, None],
                                                         f[:, :, t, None], c, n, m)
            hs.append(h)
        return torch.stack(hs, 2), c, n, m

    def seq(q, k, v, i, f, c, n, m):
        h, (c, n, m) = mk.mlstm_recurrent_sequence__b200(q, k, v, i, f, c, n, m, return_last_states=True)
        return h, c, n, m

    for fun in (loop, seq):
        eager = fun(q, k, v, i, f, c, n, m)
        compiled = torch.compile(fun, fullgraph=True)(q, k, v, i, f, c, n, m)
        for a, b in zip(eager, compiled):
            assert torch.equal(a, b)


def test_operator_registrations_pass_opcheck():
    """PyTorch's own checker: the declared schema matches what the operators do (no hidden mutation or aliasing), the
    fake implementations agree with the real outputs in shape, dtype and strides, and the autograd registration is of
    the supported kind."""
    from mlstm_kernels_b200 import _lib
    inp = case_inputs(63, 1, 2, 256, 128, 128)
    q, k, v, i, f = (to_dev(inp[n], torch.bfloat16).requires_grad_(True) for n in "qkvif")
    utils = ("test_schema", "test_faketensor", "test_autograd_registration")
    args = (q, k, v, i, f, None, None, None, 128, 1e-6, _lib.EXP, "auto", True, False)
    torch.library.opcheck(torch.ops.mlstm_b200.chunkwise_fw.default, args, test_utils=utils)
    out = torch.ops.mlstm_b200.chunkwise_fw(*args)
    bw_args = (q.detach(), k.detach(), v.detach(), i.detach(), f.detach(), None, None, None, out[1].detach(),
               out[2].detach(), out[4].detach(), torch.randn_like(out[0]).detach(), None, 128, 1e-6, _lib.EXP, "auto",
               False)
    torch.library.opcheck(torch.ops.mlstm_b200.chunkwise_bw.default, bw_args, test_utils=utils)
    g = torch.Generator(device="cuda").manual_seed(1)
    rnd = lambda *s: torch.randn(*s, device="cuda", generator=g)  # noqa: E731
    step_args = (rnd(2, 4, 128).bfloat16(), rnd(2, 4, 128).bfloat16(), rnd(2, 4, 256).bfloat16(), rnd(2, 4, 1).bfloat16(),
                 rnd(2, 4, 1).bfloat16(), rnd(2, 4, 128, 256), rnd(2, 4, 128).abs(), rnd(2, 4, 1), 1e-6, False)
    torch.library.opcheck(torch.ops.mlstm_b200.step.default, step_args, test_utils=utils)
