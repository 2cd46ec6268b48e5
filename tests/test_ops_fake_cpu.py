"""Shape and dtype inference of the custom operators (what a tracer sees), checked without a GPU: the operators'
`register_fake` functions run on fake CUDA tensors and only ask the shared library host-side questions."""

import pytest
import torch
from torch._subclasses.fake_tensor import FakeTensorMode

import mlstm_kernels_b200  # noqa: F401  (registers the operators)
from mlstm_kernels_b200 import _lib


@pytest.mark.parametrize("dtype,dims,S,want_last", [(torch.bfloat16, (256, 512), 1000, True),
                                                    (torch.bfloat16, (96, 192), 384, False),
                                                    (torch.float32, (64, 128), 256, True)])
def test_chunkwise_operator_output_shapes(dtype, dims, S, want_last):
    B, NH, (DHQK, DHHV) = 2, 3, dims
    with FakeTensorMode():
        q, k = (torch.empty(B, NH, S, DHQK, dtype=dtype, device="cuda") for _ in range(2))
        v = torch.empty(B, NH, S, DHHV, dtype=dtype, device="cuda")
        i, f = (torch.empty(B, NH, S, dtype=dtype, device="cuda") for _ in range(2))
        out = torch.ops.mlstm_b200.chunkwise_fw(q, k, v, i, f, None, None, None, 64, 1e-6, _lib.EXP, "auto", want_last,
                                                False)
        H, n_out, m_out, c_states, ws, c_last, n_last, m_last = out
        tensor_cores = dtype != torch.float32
        L = 128 if tensor_cores else 64
        assert H.shape == (B, NH, S, DHHV) and H.dtype == dtype
        assert n_out.shape == m_out.shape == (B, NH, S) and n_out.dtype == torch.float32
        assert c_states.shape == (B, NH, -(-S // L) + 1, DHQK, DHHV)
        assert c_states.dtype == (dtype if tensor_cores else torch.float32)
        assert ws.dtype == torch.uint8 and ws.numel() >= 256
        if want_last:
            assert c_last.shape == (B, NH, DHQK, DHHV) and n_last.shape == (B, NH, DHQK) and m_last.shape == (B, NH, 1)
        else:
            assert c_last.numel() == n_last.numel() == m_last.numel() == 0
        dh = torch.empty_like(H)
        grads = torch.ops.mlstm_b200.chunkwise_bw(q, k, v, i, f, None, None, None, n_out, m_out, ws, dh, None, 64,
                                                  1e-6, _lib.EXP, "auto", False)
        assert [g.shape for g in grads[:3]] == [q.shape, k.shape, v.shape]
        assert grads[3].shape == grads[4].shape == (B, NH, S) and grads[3].dtype == torch.float32
        assert grads[5].numel() == 0


def test_decode_operator_output_shapes():
    B, NH, DHQK, DHHV, T = 2, 4, 128, 256, 5
    with FakeTensorMode():
        mk_t = lambda *s, dt=torch.bfloat16: torch.empty(*s, dtype=dt, device="cuda")  # noqa: E731
        c, n, m = mk_t(B, NH, DHQK, DHHV, dt=torch.float32), mk_t(B, NH, DHQK, dt=torch.float32), mk_t(B, NH, 1, dt=torch.float32)
        h, c2, n2, m2 = torch.ops.mlstm_b200.step(mk_t(B, NH, DHQK), mk_t(B, NH, DHQK), mk_t(B, NH, DHHV),
                                                  mk_t(B, NH, 1), mk_t(B, NH, 1), c, n, m, 1e-6, False)
        assert h.shape == (B, NH, DHHV) and h.dtype == torch.bfloat16
        assert (c2.shape, n2.shape, m2.shape) == (c.shape, n.shape, m.shape) and c2.dtype == torch.float32
        h, c2, n2, m2 = torch.ops.mlstm_b200.step_sequence(mk_t(B, NH, T, DHQK), mk_t(B, NH, T, DHQK),
                                                           mk_t(B, NH, T, DHHV), mk_t(B, NH, T), mk_t(B, NH, T),
                                                           None, None, None, 1e-6)
        assert h.shape == (B, NH, T, DHHV) and c2.shape == (B, NH, DHQK, DHHV) and m2.shape == (B, NH, 1)
