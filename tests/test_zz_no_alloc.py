"""The allocation-free forward entry point (mlstm_b200_chunkwise_fw_static), called through the C ABI.

It exists for hosts that cannot call cudaMalloc while they run (all GPU memory already handed to their own
pool, or allocator calls banned from the hot loop): its scratch is a fixed array inside the library.  The
test checks that it returns exactly what the regular entry point returns, on two calls in a row (the second
call finds the array as the first one left it), and that cases beyond the built-in limit are refused.
This file sorts last on purpose: a run that stops at the first failure has then already run everything else.
"""

import ctypes as C

import pytest
import torch

from inputs import max_rel_err
from mlstm_kernels_b200 import _lib
from util_gpu import case_inputs, npy, to_dev

pytestmark = pytest.mark.gpu


def _buffers(B, NH, S, DHQK, DHHV, L, sdt):
    dev = "cuda"
    NC = S // L
    return dict(
        h=torch.empty(B, NH, S, DHHV, dtype=torch.bfloat16, device=dev),
        n_out=torch.empty(B, NH, S, device=dev), m_out=torch.empty(B, NH, S, device=dev),
        c_states=torch.empty(B, NH, NC + 1, DHQK, DHHV, dtype=sdt, device=dev),
        n_states=torch.zeros(B, NH, NC + 1, DHQK, device=dev), m_states=torch.empty(B, NH, NC + 1, device=dev),
        c_last=torch.empty(B, NH, DHQK, DHHV, device=dev), n_last=torch.zeros(B, NH, DHQK, device=dev),
        m_last=torch.empty(B, NH, 1, device=dev))


def _call(lib, static, tensors, out, dims, ws=None):
    q, k, v, i, f = tensors
    p = _lib.ptr
    head = [p(q), p(k), p(v), p(i), p(f), None, None, None, p(out["h"]), p(out["n_out"]), p(out["m_out"]),
            p(out["c_states"]), p(out["n_states"]), p(out["m_states"]), p(out["c_last"]), p(out["n_last"]),
            p(out["m_last"])]
    tail = [*dims, _lib.BF16, _lib.BF16, _lib.EXP, _lib.IMPL["auto"], 1e-6, _lib.stream_handle(q.device)]
    if static:
        return lib.mlstm_b200_chunkwise_fw_static(*head, *tail)
    return lib.mlstm_b200_chunkwise_fw(*head, p(ws), ws.numel(), *tail)


def test_static_scratch_forward_matches_regular_entry_point_twice():
    lib = _lib.load()
    B, NH, S, DHQK, DHHV, L = 2, 2, 512, 128, 128, 128
    dims = (B, NH, S, DHQK, DHHV, L)
    sdt = _lib.code_dtype(lib.mlstm_b200_chunkwise_state_dtype(S, DHQK, DHHV, L, _lib.BF16, 0))
    assert lib.mlstm_b200_static_scratch_bytes() == 8 << 20
    for seed in (101, 102):  # two calls in a row, different data
        inp = case_inputs(seed, B, NH, S, DHQK, DHHV)
        tensors = [to_dev(inp[n], torch.bfloat16) for n in "qkvif"]
        ws_bytes = lib.mlstm_b200_chunkwise_workspace_bytes(*dims, _lib.BF16, _lib.EXP, 0, 0)
        ws = torch.empty(ws_bytes, dtype=torch.uint8, device="cuda")
        ref, got = _buffers(*dims, sdt), _buffers(*dims, sdt)
        assert _call(lib, False, tensors, ref, dims, ws) == 0
        assert _call(lib, True, tensors, got, dims) == 0
        torch.cuda.synchronize()
        for name in ref:
            assert max_rel_err(npy(got[name].float()), npy(ref[name].float())) <= 1e-6, name
    assert _lib.device_status() == 0


def test_static_warmup_then_calls_take_no_driver_memory():
    """After mlstm_b200_static_warmup() and one call, a further call leaves the driver's free-memory figure where it
    was: the array and the kernels' code were materialised up front, the call itself allocates nothing."""
    lib = _lib.load()
    assert lib.mlstm_b200_static_warmup() == 0
    B, NH, S, DHQK, DHHV, L = 1, 2, 256, 128, 128, 128
    dims = (B, NH, S, DHQK, DHHV, L)
    sdt = _lib.code_dtype(lib.mlstm_b200_chunkwise_state_dtype(S, DHQK, DHHV, L, _lib.BF16, 0))
    inp = case_inputs(103, B, NH, S, DHQK, DHHV)
    tensors = [to_dev(inp[n], torch.bfloat16) for n in "qkvif"]
    out = _buffers(*dims, sdt)
    assert _call(lib, True, tensors, out, dims) == 0
    torch.cuda.synchronize()
    free_before, _ = torch.cuda.mem_get_info()
    assert _call(lib, True, tensors, out, dims) == 0
    torch.cuda.synchronize()
    free_after, _ = torch.cuda.mem_get_info()
    assert free_after == free_before
    assert _lib.device_status() == 0


def test_static_scratch_rejects_cases_beyond_its_limit():
    lib = _lib.load()
    B, NH, S, DHQK, DHHV, L = 16, 16, 8192, 128, 128, 128   # 2M token-heads: needs ~34 MB of scratch
    dims = (B, NH, S, DHQK, DHHV, L)
    assert lib.mlstm_b200_chunkwise_workspace_bytes(*dims, _lib.BF16, _lib.EXP, 0, 0) > lib.mlstm_b200_static_scratch_bytes()
    null = C.c_void_p(None)
    rc = lib.mlstm_b200_chunkwise_fw_static(*([null] * 17), *dims, _lib.BF16, _lib.BF16, _lib.EXP, 0, 1e-6, null)
    assert rc == -5  # MLSTM_ERR_WORKSPACE: refused before any pointer is touched or kernel launched
    assert b"workspace" in lib.mlstm_b200_error_string(rc)
