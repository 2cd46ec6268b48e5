"""PyTorch-facing recurrent decode kernels backed by libmlstm_b200.so.

`mlstm_recurrent_step__b200` keeps the signature of mlstm_recurrent_step__triton
(mlstm_kernels/torch/recurrent/triton_step.py:130-158); `mlstm_recurrent_sequence__b200` that of the
sequence kernels (mlstm_kernels/torch/recurrent/native_sequence.py:125-170)."""

from __future__ import annotations

import torch

from . import _lib


def mlstm_recurrent_step__b200_fw(
    matC_old: torch.Tensor,  # (B, NH, DHQK, DHHV)
    vecN_old: torch.Tensor,  # (B, NH, DHQK)
    scaM_old: torch.Tensor,  # (B, NH, 1)
    vecQ: torch.Tensor,  # (B, NH, DHQK)
    vecK: torch.Tensor,  # (B, NH, DHQK)
    vecV: torch.Tensor,  # (B, NH, DHHV)
    scaI: torch.Tensor,  # (B, NH, 1)
    scaF: torch.Tensor,  # (B, NH, 1)
    matC_new: torch.Tensor = None,
    vecN_new: torch.Tensor = None,
    scaM_new: torch.Tensor = None,
    eps: float = 1e-6,
    dtype_state: torch.dtype = torch.float32,
    **kwargs,
):
    _lib.require_cuda(matC_old, vecN_old, scaM_old, vecQ, vecK, vecV, scaI, scaF)
    lib = _lib.load()
    B, NH, DHQK = vecQ.shape
    DHHV = vecV.shape[-1]
    assert vecQ.shape == vecK.shape, "q and k must have the same shape"
    assert matC_old.shape == (B, NH, DHQK, DHHV), f"matC_old has wrong shape, got {matC_old.shape}"
    assert vecN_old.shape == (B, NH, DHQK), f"vecN_old has wrong shape, got {vecN_old.shape}"
    assert scaM_old.shape == (B, NH, 1), f"scaM_old has wrong shape, got {scaM_old.shape}"
    assert scaI.shape == (B, NH, 1), f"scaI has wrong shape, got {scaI.shape}"
    assert scaF.shape == (B, NH, 1), f"scaF has wrong shape, got {scaF.shape}"
    if dtype_state not in (torch.float32, torch.bfloat16):
        raise ValueError(f"Unsupported state dtype {dtype_state}.")
    dt = _lib.dtype_code(vecQ.dtype)
    q, k, v = vecQ.contiguous(), vecK.to(vecQ.dtype).contiguous(), vecV.to(vecQ.dtype).contiguous()
    gi, gf = scaI.to(vecQ.dtype).contiguous(), scaF.to(vecQ.dtype).contiguous()
    c, n, m = (t.to(dtype_state).contiguous() for t in (matC_old, vecN_old, scaM_old))
    if matC_new is None:
        assert vecN_new is None and scaM_new is None, "Initial states must be provided together."
        matC_new, vecN_new, scaM_new = torch.empty_like(c), torch.empty_like(n), torch.empty_like(m)
    else:
        assert vecN_new is not None and scaM_new is not None, "Initial states must be provided together."
        for t in (matC_new, vecN_new, scaM_new):
            if t.dtype != dtype_state or not t.is_contiguous():
                raise ValueError("output state tensors must be contiguous and of dtype_state")
    h = torch.empty_like(v)
    dev = q.device
    with torch.cuda.device(dev):
        rc = lib.mlstm_b200_step(_lib.ptr(q), _lib.ptr(k), _lib.ptr(v), _lib.ptr(gi), _lib.ptr(gf),
                                 _lib.ptr(c), _lib.ptr(n), _lib.ptr(m), _lib.ptr(h),
                                 _lib.ptr(matC_new), _lib.ptr(vecN_new), _lib.ptr(scaM_new),
                                 B, NH, DHQK, DHHV, dt, _lib.dtype_code(dtype_state), float(eps),
                                 _lib.stream_handle(dev))
    _lib.check(rc, "mlstm_b200_step")
    return h, (matC_new, vecN_new, scaM_new)


def mlstm_recurrent_step__b200(
    q: torch.Tensor,  # (B, NH, DHQK)
    k: torch.Tensor,  # (B, NH, DHQK)
    v: torch.Tensor,  # (B, NH, DHHV)
    i: torch.Tensor,  # (B, NH, 1)
    f: torch.Tensor,  # (B, NH, 1)
    c: torch.Tensor,  # (B, NH, DHQK, DHHV)
    n: torch.Tensor,  # (B, NH, DHQK)
    m: torch.Tensor,  # (B, NH, 1)
    eps: float = 1e-6,
    dtype_state: torch.dtype = torch.float32,
    **kwargs,
) -> tuple[torch.Tensor, tuple[torch.Tensor, torch.Tensor, torch.Tensor]]:
    """One mLSTM decode step: returns h (B,NH,DHHV) and the new (C, n, m); the old states are untouched."""
    return mlstm_recurrent_step__b200_fw(matC_old=c, vecN_old=n, scaM_old=m, vecQ=q, vecK=k, vecV=v, scaI=i,
                                         scaF=f, eps=eps, dtype_state=dtype_state, **kwargs)


def mlstm_recurrent_sequence__b200(
    q: torch.Tensor,  # (B, NH, S, DHQK)
    k: torch.Tensor,
    v: torch.Tensor,  # (B, NH, S, DHHV)
    i: torch.Tensor,  # (B, NH, S)
    f: torch.Tensor,
    c_initial: torch.Tensor = None,
    n_initial: torch.Tensor = None,
    m_initial: torch.Tensor = None,
    return_last_states: bool = False,
    eps: float = 1e-6,
    dtype_state: torch.dtype = torch.float32,
    **kwargs,
):
    """S decode steps in ONE launch with the state held in registers (replaces the per-token Python loop)."""
    _lib.require_cuda(q, k, v, i, f)
    lib = _lib.load()
    B, NH, S, DHQK = q.shape
    DHHV = v.shape[-1]
    dt = _lib.dtype_code(q.dtype)
    q, k, v = q.contiguous(), k.to(q.dtype).contiguous(), v.to(q.dtype).contiguous()
    gi, gf = i.to(q.dtype).contiguous(), f.to(q.dtype).contiguous()
    f32 = lambda t: None if t is None else t.to(torch.float32).contiguous()  # noqa: E731
    c0, n0, m0 = f32(c_initial), f32(n_initial), f32(m_initial)
    dev = q.device
    h = torch.empty_like(v)
    c_new = torch.empty((B, NH, DHQK, DHHV), dtype=torch.float32, device=dev)
    n_new = torch.empty((B, NH, DHQK), dtype=torch.float32, device=dev)
    m_new = torch.empty((B, NH, 1), dtype=torch.float32, device=dev)
    with torch.cuda.device(dev):
        rc = lib.mlstm_b200_step_sequence(_lib.ptr(q), _lib.ptr(k), _lib.ptr(v), _lib.ptr(gi), _lib.ptr(gf),
                                          _lib.ptr(c0), _lib.ptr(n0), _lib.ptr(m0), _lib.ptr(h),
                                          _lib.ptr(c_new), _lib.ptr(n_new), _lib.ptr(m_new),
                                          B, NH, S, DHQK, DHHV, dt, float(eps), _lib.stream_handle(dev))
    _lib.check(rc, "mlstm_b200_step_sequence")
    if return_last_states:
        return h, (c_new.to(dtype_state), n_new.to(dtype_state), m_new.to(dtype_state))
    return h
