"""PyTorch-facing recurrent decode kernels backed by libmlstm_b200.so.

`mlstm_recurrent_step__b200` keeps the signature of mlstm_recurrent_step__triton
(mlstm_kernels/torch/recurrent/triton_step.py:130-158); `mlstm_recurrent_sequence__b200` that of the
sequence kernels (mlstm_kernels/torch/recurrent/native_sequence.py:125-170).

A decode step at small batch is a few microseconds of device time, so the host side of the step is written
to do as little as possible: tensors that already have the expected element type and layout are passed
through untouched (no `.to()`, no `.contiguous()`), the gate pre-activations keep their own element type
(the kernel widens them to f32, as mlstm_kernels/triton/recurrent/fw_step_fused.py:88-94 does), and the
device guard is skipped when the tensors' device is already current.
"""

from __future__ import annotations

import torch

from . import _lib, _ops

_STATE_DTYPES = (torch.float32, torch.bfloat16)

# cheapest routes to the current device ordinal and the current stream's handle
_current_device = getattr(torch._C, "_cuda_getDevice", torch.cuda.current_device)
_raw_stream_c = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _raw_stream(device_index: int) -> int:
    if _raw_stream_c is not None:
        return _raw_stream_c(device_index)
    return torch.cuda.current_stream(device_index).cuda_stream


_STEP_FN = None


def _step_fn():
    global _STEP_FN
    if _STEP_FN is None:
        _STEP_FN = _lib.load().mlstm_b200_step
    return _STEP_FN


def _conform(t: torch.Tensor, dtype: torch.dtype) -> torch.Tensor:
    if t.dtype is not dtype:
        t = t.to(dtype)
    return t if t.is_contiguous() else t.contiguous()


def _gate(t: torch.Tensor) -> torch.Tensor:
    """Gate pre-activations in one of the kernel's gate element types, contiguous."""
    if t.dtype not in _lib._DTYPE_CODE:
        t = t.to(torch.float32)
    return t if t.is_contiguous() else t.contiguous()


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
    vecH_out: torch.Tensor = None,  # optional caller-owned output (B, NH, DHHV) in q's dtype
    validate: bool = True,
    **kwargs,
):
    """One decode step.  `validate=False` is for decode loops that own all their buffers: every tensor (the new-state
    and `vecH_out` buffers included) must then be a contiguous CUDA tensor of the expected shape and element type on
    the current device; nothing is checked or converted and the call costs little more than the launch itself."""
    if not validate:
        B, NH, DHQK = vecQ.shape
        codes = _lib._DTYPE_CODE
        rc = _step_fn()(vecQ.data_ptr(), vecK.data_ptr(), vecV.data_ptr(), scaI.data_ptr(), scaF.data_ptr(),
                        matC_old.data_ptr(), vecN_old.data_ptr(), scaM_old.data_ptr(), vecH_out.data_ptr(),
                        matC_new.data_ptr(), vecN_new.data_ptr(), scaM_new.data_ptr(), B, NH, DHQK,
                        vecV.shape[-1], codes[vecQ.dtype], codes[scaI.dtype], codes[dtype_state], eps,
                        _raw_stream(vecQ.device.index))
        if rc != 0:
            _lib.check(rc, "mlstm_b200_step")
        return vecH_out, (matC_new, vecN_new, scaM_new)
    if not (vecQ.is_cuda and matC_old.is_cuda):
        raise RuntimeError("mlstm_kernels_b200 kernels run on CUDA tensors only (there is no CPU fallback)")
    B, NH, DHQK = vecQ.shape
    DHHV = vecV.shape[-1]
    assert vecQ.shape == vecK.shape, "q and k must have the same shape"
    assert matC_old.shape == (B, NH, DHQK, DHHV), f"matC_old has wrong shape, got {matC_old.shape}"
    assert vecN_old.shape == (B, NH, DHQK), f"vecN_old has wrong shape, got {vecN_old.shape}"
    assert scaM_old.shape == (B, NH, 1), f"scaM_old has wrong shape, got {scaM_old.shape}"
    assert scaI.shape == (B, NH, 1), f"scaI has wrong shape, got {scaI.shape}"
    assert scaF.shape == (B, NH, 1), f"scaF has wrong shape, got {scaF.shape}"
    if dtype_state not in _STATE_DTYPES:
        raise ValueError(f"Unsupported state dtype {dtype_state}.")
    qdt = vecQ.dtype
    codes = _lib._DTYPE_CODE
    dt = codes.get(qdt)
    if dt is None:
        raise ValueError(f"Unsupported kernel dtype {qdt}.")
    # tensors that already conform are passed through untouched
    q = vecQ if vecQ.is_contiguous() else vecQ.contiguous()
    k = vecK if (vecK.dtype is qdt and vecK.is_contiguous()) else _conform(vecK, qdt)
    v = vecV if (vecV.dtype is qdt and vecV.is_contiguous()) else _conform(vecV, qdt)
    gi = scaI if (scaI.dtype in codes and scaI.is_contiguous()) else _gate(scaI)
    gdt = gi.dtype
    gf = scaF if (scaF.dtype is gdt and scaF.is_contiguous()) else _conform(scaF, gdt)
    c = matC_old if (matC_old.dtype is dtype_state and matC_old.is_contiguous()) else _conform(matC_old, dtype_state)
    n = vecN_old if (vecN_old.dtype is dtype_state and vecN_old.is_contiguous()) else _conform(vecN_old, dtype_state)
    m = scaM_old if (scaM_old.dtype is dtype_state and scaM_old.is_contiguous()) else _conform(scaM_old, dtype_state)
    if matC_new is None:
        assert vecN_new is None and scaM_new is None, "Initial states must be provided together."
        matC_new, vecN_new, scaM_new = torch.empty_like(c), torch.empty_like(n), torch.empty_like(m)
    else:
        assert vecN_new is not None and scaM_new is not None, "Initial states must be provided together."
        for t in (matC_new, vecN_new, scaM_new):
            if t.dtype is not dtype_state or not t.is_contiguous():
                raise ValueError("output state tensors must be contiguous and of dtype_state")
    if vecH_out is None:
        h = torch.empty_like(v)
    else:
        h = vecH_out
        if h.dtype is not qdt or h.shape != v.shape or not h.is_contiguous():
            raise ValueError("vecH_out must be a contiguous (B, NH, DHHV) tensor of q's dtype")
    # raw addresses go to ctypes as plain integers (the argument types are declared once in _lib.SIGNATURES)
    dev_index = q.device.index
    if _current_device() == dev_index:
        rc = _step_fn()(q.data_ptr(), k.data_ptr(), v.data_ptr(), gi.data_ptr(), gf.data_ptr(), c.data_ptr(),
                        n.data_ptr(), m.data_ptr(), h.data_ptr(), matC_new.data_ptr(), vecN_new.data_ptr(),
                        scaM_new.data_ptr(), B, NH, DHQK, DHHV, dt, codes[gdt], codes[dtype_state], eps,
                        _raw_stream(dev_index))
    else:
        with torch.cuda.device(q.device):
            rc = _step_fn()(q.data_ptr(), k.data_ptr(), v.data_ptr(), gi.data_ptr(), gf.data_ptr(), c.data_ptr(),
                            n.data_ptr(), m.data_ptr(), h.data_ptr(), matC_new.data_ptr(), vecN_new.data_ptr(),
                            scaM_new.data_ptr(), B, NH, DHQK, DHHV, dt, codes[gdt], codes[dtype_state], eps,
                            _raw_stream(dev_index))
    if rc != 0:
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
    if torch.compiler.is_compiling():   # a tracer is watching: go through the custom operator
        if dtype_state not in _STATE_DTYPES:
            raise ValueError(f"Unsupported state dtype {dtype_state}.")
        h, c_new, n_new, m_new = _ops.step(q, k, v, i, f, c, n, m, eps, dtype_state is torch.bfloat16)
        return h, (c_new, n_new, m_new)
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
    if torch.compiler.is_compiling():   # a tracer is watching: go through the custom operator
        h, c_new, n_new, m_new = _ops.step_sequence(q, k, v, i, f, c_initial, n_initial, m_initial, eps)
        if return_last_states:
            return h, (c_new.to(dtype_state), n_new.to(dtype_state), m_new.to(dtype_state))
        return h
    _lib.require_cuda(q, k, v, i, f)
    lib = _lib.load()
    B, NH, S, DHQK = q.shape
    DHHV = v.shape[-1]
    dt = _lib.dtype_code(q.dtype)
    q, k, v = q.contiguous(), _conform(k, q.dtype), _conform(v, q.dtype)
    gi = _gate(i)
    gf = _conform(f, gi.dtype)
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
                                          B, NH, S, DHQK, DHHV, dt, _lib.dtype_code(gi.dtype), float(eps),
                                          _lib.stream_handle(dev))
    _lib.check(rc, "mlstm_b200_step_sequence")
    if return_last_states:
        return h, (c_new.to(dtype_state), n_new.to(dtype_state), m_new.to(dtype_state))
    return h
