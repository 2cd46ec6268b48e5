"""The kernels as PyTorch custom operators, for callers that trace their models (torch.compile).

The eager shims of chunkwise.py / recurrent.py talk to the shared library through ctypes, which a tracer can neither
follow nor skip.  Wrapped as `torch.library` operators the same calls become opaque nodes of the traced graph: shapes
and dtypes of the outputs come from the `register_fake` functions below (which only ask the library host-side
questions - chunk size, state element type, workspace size), gradients from `register_autograd`.  The reference's
Triton kernels are traceable in the same sense (its benchmark compiles whole models:
mlstm_kernels/utils/benchmark/benchmarks/interface.py:94-95).

The public functions switch to these operators only while a trace is being taken (`torch.compiler.is_compiling()`);
eager calls keep the direct path, which costs less per call.  Outputs an operator does not produce in some mode
(the last states without `want_last`, dC_initial without `want_dc0`) are empty tensors: an operator returns a fixed
number of tensors.
"""

from __future__ import annotations

from typing import Optional

import torch
from torch import Tensor

from . import _lib

_F32 = torch.float32


def _empty(like: Tensor) -> Tensor:
    return like.new_empty((0,), dtype=_F32)


def _opt(t: Tensor) -> Optional[Tensor]:
    return None if t is None or t.numel() == 0 else t


# ---- chunkwise forward ------------------------------------------------------------------------------------------
@torch.library.custom_op("mlstm_b200::chunkwise_fw", mutates_args=(), device_types="cuda")
def chunkwise_fw(q: Tensor, k: Tensor, v: Tensor, i: Tensor, f: Tensor, c_initial: Optional[Tensor],
                 n_initial: Optional[Tensor], m_initial: Optional[Tensor], chunk_size: int, eps: float, variant: int,
                 impl: str, want_last: bool, keep_states: bool
                 ) -> tuple[Tensor, Tensor, Tensor, Tensor, Tensor, Tensor, Tensor, Tensor]:
    """(H, n_out, m_out, C_states, workspace, C_last, n_last, m_last); `keep_states` only tells the autograd
    registration whether the backward gets the per-chunk states or recomputes them."""
    from .chunkwise import chunkwise_fw_raw, resolve_chunk_size
    L = resolve_chunk_size(q, v, chunk_size, impl)
    out = chunkwise_fw_raw(q, k, v, i, f, c_initial, n_initial, m_initial if variant == _lib.EXP else None,
                           chunk_size=L, eps=eps, variant=variant, impl=impl, want_last=want_last)
    last = (out["C_last"], out["n_last"], out["m_last"]) if want_last else (_empty(q), _empty(q), _empty(q))
    return (out["H"], out["n_out"], out["m_out"], out["C_states"], out["workspace"]) + last


@chunkwise_fw.register_fake
def _(q, k, v, i, f, c_initial, n_initial, m_initial, chunk_size, eps, variant, impl, want_last, keep_states):
    from .chunkwise import resolve_chunk_size
    lib = _lib.load()
    B, NH, S, DHQK = q.shape
    DHHV = v.shape[-1]
    L = resolve_chunk_size(q, v, chunk_size, impl)
    NC = -(-S // L)
    dt, im = _lib.dtype_code(q.dtype), _lib.IMPL[impl]
    sdt = _lib.code_dtype(lib.mlstm_b200_chunkwise_state_dtype(S, DHQK, DHHV, L, dt, im))
    ws = lib.mlstm_b200_chunkwise_workspace_bytes(B, NH, S, DHQK, DHHV, L, dt, variant, im, 0)
    last = ((q.new_empty((B, NH, DHQK, DHHV), dtype=_F32), q.new_empty((B, NH, DHQK), dtype=_F32),
             q.new_empty((B, NH, 1), dtype=_F32)) if want_last else (_empty(q), _empty(q), _empty(q)))
    return (q.new_empty((B, NH, S, DHHV)), q.new_empty((B, NH, S), dtype=_F32), q.new_empty((B, NH, S), dtype=_F32),
            q.new_empty((B, NH, NC + 1, DHQK, DHHV), dtype=sdt), q.new_empty((max(ws, 256),), dtype=torch.uint8)) + last


# ---- chunkwise backward -----------------------------------------------------------------------------------------
@torch.library.custom_op("mlstm_b200::chunkwise_bw", mutates_args=(), device_types="cuda")
def chunkwise_bw(q: Tensor, k: Tensor, v: Tensor, i: Tensor, f: Tensor, m_initial: Optional[Tensor],
                 c_initial: Optional[Tensor], c_states: Optional[Tensor], n_out: Tensor, m_out: Tensor,
                 workspace: Tensor, dh: Tensor, dc_last: Optional[Tensor], chunk_size: int, eps: float, variant: int,
                 impl: str, want_dc0: bool) -> tuple[Tensor, Tensor, Tensor, Tensor, Tensor, Tensor]:
    """(dq, dk, dv, di, df, dc_initial).  c_states = None: the per-chunk states are recomputed (from c_initial)."""
    from .chunkwise import chunkwise_bw_raw, resolve_chunk_size
    L = resolve_chunk_size(q, v, chunk_size, impl)
    dq, dk, dv, di, df, dc0 = chunkwise_bw_raw(
        q, k, v, i, f, m_initial if variant == _lib.EXP else None, c_states, n_out, dh, dc_last, chunk_size=L,
        eps=eps, variant=variant, impl=impl, want_dc_initial=want_dc0, m_out=m_out, fw_workspace=workspace,
        recompute_c_initial=c_initial)
    return dq, dk, dv, di, df, dc0 if want_dc0 else _empty(q)


@chunkwise_bw.register_fake
def _(q, k, v, i, f, m_initial, c_initial, c_states, n_out, m_out, workspace, dh, dc_last, chunk_size, eps, variant,
      impl, want_dc0):
    B, NH, S, DHQK = q.shape
    dc0 = q.new_empty((B, NH, DHQK, v.shape[-1]), dtype=_F32) if want_dc0 else _empty(q)
    return (torch.empty_like(q, memory_format=torch.contiguous_format),
            torch.empty_like(k, memory_format=torch.contiguous_format),
            torch.empty_like(v, memory_format=torch.contiguous_format),
            q.new_empty((B, NH, S), dtype=_F32), q.new_empty((B, NH, S), dtype=_F32), dc0)


def _fw_setup_context(ctx, inputs, output):
    q, k, v, i, f, c_initial, n_initial, m_initial, chunk_size, eps, variant, impl, want_last, keep_states = inputs
    _, n_out, m_out, c_states, workspace = output[:5]
    ctx.cfg = (chunk_size, eps, variant, impl, c_initial is not None, n_initial is not None, m_initial is not None,
               None if c_initial is None else c_initial.dtype, None if n_initial is None else n_initial.dtype,
               (q.shape[0], q.shape[1], q.shape[3]), i.dtype, f.dtype)
    ctx.save_for_backward(q, k, v, i, f, None if keep_states else c_initial, m_initial,
                          c_states if keep_states else None, n_out, m_out, workspace)


def _fw_backward(ctx, dH, _dn_out, _dm_out, _dc_states, _dws, dC_last, _dn_last, _dm_last):
    q, k, v, i, f, c_initial, m_initial, c_states, n_out, m_out, workspace = ctx.saved_tensors
    chunk_size, eps, variant, impl, has_c0, has_n0, has_m0, c0_dtype, n0_dtype, (B, NH, DHQK), i_dtype, f_dtype = ctx.cfg
    if dH is None:
        dH = torch.zeros((B, NH, q.shape[2], v.shape[-1]), dtype=q.dtype, device=q.device)
    dq, dk, dv, di, df, dc0 = chunkwise_bw(q, k, v, i, f, m_initial, c_initial, c_states, n_out, m_out, workspace,
                                          dH.contiguous(), _opt(dC_last), chunk_size, eps, variant, impl, has_c0)
    dn0 = torch.zeros((B, NH, DHQK), dtype=n0_dtype, device=q.device) if has_n0 else None
    dm0 = torch.zeros((B, NH, 1), dtype=m_initial.dtype, device=q.device) if has_m0 else None
    return (dq, dk, dv, di.to(i_dtype), df.to(f_dtype), dc0.to(c0_dtype) if has_c0 else None, dn0, dm0,
            None, None, None, None, None, None)


torch.library.register_autograd("mlstm_b200::chunkwise_fw", _fw_backward, setup_context=_fw_setup_context)


def chunkwise_traced(q, k, v, i, f, c_initial, n_initial, m_initial, return_last_states, eps, chunk_size, impl,
                     recompute_states_in_bw, autocast_kernel_dtype, variant):
    """What the public chunkwise functions do while a trace is being taken: the autocast rule of
    torch.amp.custom_fwd(cast_inputs=...) written out (inside an autocast region floating-point inputs are cast to
    `autocast_kernel_dtype` and the kernel runs with autocast off), then the operator."""
    if torch.is_autocast_enabled("cuda"):
        cast = lambda t: t.to(autocast_kernel_dtype) if (t is not None and t.is_floating_point()) else t  # noqa: E731
        q, k, v, i, f, c_initial, n_initial, m_initial = (cast(t) for t in (q, k, v, i, f, c_initial, n_initial,
                                                                             m_initial))
        with torch.autocast("cuda", enabled=False):
            out = chunkwise_fw(q, k, v, i, f, c_initial, n_initial, m_initial, chunk_size, eps, variant, impl,
                               return_last_states, not recompute_states_in_bw)
    else:
        out = chunkwise_fw(q, k, v, i, f, c_initial, n_initial, m_initial, chunk_size, eps, variant, impl,
                           return_last_states, not recompute_states_in_bw)
    return out[0], out[5], out[6], out[7]


# ---- decode -----------------------------------------------------------------------------------------------------
@torch.library.custom_op("mlstm_b200::step", mutates_args=(), device_types="cuda")
def step(q: Tensor, k: Tensor, v: Tensor, i: Tensor, f: Tensor, c: Tensor, n: Tensor, m: Tensor, eps: float,
         state_is_bf16: bool) -> tuple[Tensor, Tensor, Tensor, Tensor]:
    from .recurrent import mlstm_recurrent_step__b200_fw
    h, (c_new, n_new, m_new) = mlstm_recurrent_step__b200_fw(
        c, n, m, q, k, v, i, f, eps=eps, dtype_state=torch.bfloat16 if state_is_bf16 else _F32)
    return h, c_new, n_new, m_new


@step.register_fake
def _(q, k, v, i, f, c, n, m, eps, state_is_bf16):
    sdt = torch.bfloat16 if state_is_bf16 else _F32
    return (torch.empty_like(v, memory_format=torch.contiguous_format), c.new_empty(c.shape, dtype=sdt),
            n.new_empty(n.shape, dtype=sdt), m.new_empty(m.shape, dtype=sdt))


@torch.library.custom_op("mlstm_b200::step_sequence", mutates_args=(), device_types="cuda")
def step_sequence(q: Tensor, k: Tensor, v: Tensor, i: Tensor, f: Tensor, c_initial: Optional[Tensor],
                  n_initial: Optional[Tensor], m_initial: Optional[Tensor], eps: float
                  ) -> tuple[Tensor, Tensor, Tensor, Tensor]:
    from .recurrent import mlstm_recurrent_sequence__b200
    h, (c_new, n_new, m_new) = mlstm_recurrent_sequence__b200(q, k, v, i, f, c_initial, n_initial, m_initial,
                                                              return_last_states=True, eps=eps)
    return h, c_new, n_new, m_new


@step_sequence.register_fake
def _(q, k, v, i, f, c_initial, n_initial, m_initial, eps):
    B, NH, S, DHQK = q.shape
    DHHV = v.shape[-1]
    return (torch.empty_like(v, memory_format=torch.contiguous_format), q.new_empty((B, NH, DHQK, DHHV), dtype=_F32),
            q.new_empty((B, NH, DHQK), dtype=_F32), q.new_empty((B, NH, 1), dtype=_F32))
