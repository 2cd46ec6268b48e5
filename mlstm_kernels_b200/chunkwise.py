"""PyTorch-facing chunkwise mLSTM kernels backed by libmlstm_b200.so.

`mlstm_chunkwise__b200_xl_chunk` and `mlstm_siging_chunkwise__b200_xl_chunk` keep the signatures,
return conventions and error behaviour of the reference's
mlstm_chunkwise__xl_chunk (mlstm_kernels/torch/chunkwise/triton_xl_chunk/fwbw.py:244-300) and
mlstm_siging_chunkwise__xl_chunk (mlstm_kernels/torch/chunkwise/triton_xl_chunk_siging/fwbw.py:211-269),
so they can be registered as chunkwise kernels of the reference's mLSTMBackend.
The Triton tuning keyword arguments are accepted and ignored.
"""

from __future__ import annotations

import os

import torch
from torch.amp import custom_bwd, custom_fwd

from . import _lib, _ops

# MLSTM_B200_CHECK_STATUS=1: after every backward, synchronise and raise if a bounded wait of the tcgen05 kernels
# ran out (their results are then invalid).  Off by default because the check waits for the device.
_CHECK_STATUS = os.environ.get("MLSTM_B200_CHECK_STATUS", "0") == "1"


def _is_pow2(x: int) -> bool:
    return x > 0 and (x & (x - 1)) == 0


def select_chunk_size(sequence_length: int, target_chunk_size: int) -> int:
    """Chunk size actually used, following the reference's heuristic
    (mlstm_kernels/triton/chunkwise/kernel_param_heuristics.py:42-128): sequences shorter than 128
    are processed as one chunk; otherwise the target chunk size must divide the sequence length."""
    if sequence_length % 16 != 0:
        raise ValueError("Sequence length must be divisible by 16.")
    if target_chunk_size is None:
        target_chunk_size = 128
    if sequence_length < 128:
        if _is_pow2(sequence_length):
            return sequence_length
        if _is_pow2(target_chunk_size) and target_chunk_size >= 16 and sequence_length % target_chunk_size == 0:
            return target_chunk_size  # more permissive than the reference, which rejects this case
        raise ValueError("Sequence length must be a power of 2.")
    if not _is_pow2(target_chunk_size) or target_chunk_size < 16:
        raise ValueError(f"Chunk size {target_chunk_size} must be a power of 2 >= 16.")
    if sequence_length % target_chunk_size != 0:
        raise ValueError(
            f"Sequence length must be divisible by the target chunk size {target_chunk_size}.")
    return target_chunk_size


def tcgen05_applies(q: torch.Tensor, v: torch.Tensor, impl: str = "auto") -> bool:
    """True where the tcgen05 kernels run: bf16 or fp16, head dims multiples of 8 up to 512 (qk) / 1024 (v),
    any sequence length."""
    if impl == "simt" or not q.is_cuda or q.dtype not in _lib._DTYPE_CODE:
        return False
    lib = _lib.load()
    return bool(lib.mlstm_b200_chunkwise_has_tcgen05(q.shape[2], q.shape[3], v.shape[3], 128, _lib.dtype_code(q.dtype)))


def kernel_chunk_size(q: torch.Tensor, v: torch.Tensor, chunk_size: int, impl: str = "auto") -> int:
    """Chunk size the kernels run with.  Where the tcgen05 path applies (bf16 or fp16, head dims multiples of 8) every
    requested chunk size runs as chunks of 128, the last one ragged if the sequence length is no multiple of 128
    (H does not depend on the chunk size; the reference does the same for its inter-chunk kernel:
    chunk_size_inter = min(128, chunk_size), mlstm_kernels/triton/chunkwise/kernel_param_heuristics.py:96-121)."""
    return 128 if tcgen05_applies(q, v, impl) else chunk_size


def resolve_chunk_size(q: torch.Tensor, v: torch.Tensor, chunk_size: int, impl: str = "auto") -> int:
    """The chunk size a call runs with.  On the tcgen05 path any sequence length is accepted (no padding, no
    divisibility rule); elsewhere the reference's rules apply (select_chunk_size)."""
    if tcgen05_applies(q, v, impl):
        return 128
    return select_chunk_size(q.shape[2], chunk_size)


def _f32c(t):
    return None if t is None else t.to(torch.float32).contiguous()


def chunkwise_fw_raw(q, k, v, i, f, c_initial=None, n_initial=None, m_initial=None, *, chunk_size: int,
                     eps: float, variant: int, impl: str = "auto", want_last: bool = True):
    """Run the forward kernels.  Returns a dict with H, n_out, m_out, the per-chunk states and
    (optionally) f32 copies of the final state."""
    _lib.require_cuda(q, k, v, i, f)
    lib = _lib.load()
    B, NH, S, DHQK = q.shape
    DHHV = v.shape[-1]
    if k.shape != (B, NH, S, DHQK) or v.shape[:3] != (B, NH, S) or i.shape != (B, NH, S) or f.shape != (B, NH, S):
        raise ValueError("q, k, v, i, f have inconsistent shapes")
    if k.dtype != q.dtype or v.dtype != q.dtype:
        raise ValueError("q, k, v must share one dtype")
    if i.dtype != f.dtype:
        f = f.to(i.dtype)
    L = chunk_size
    NC = -(-S // L)   # the last chunk may be ragged on the tcgen05 path (the library refuses it elsewhere)
    dt, gdt, im = _lib.dtype_code(q.dtype), _lib.dtype_code(i.dtype), _lib.IMPL[impl]
    q, k, v, i, f = (t.contiguous() for t in (q, k, v, i, f))
    c0, n0 = _f32c(c_initial), _f32c(n_initial)
    m0 = None if m_initial is None else _f32c(m_initial).reshape(B, NH)
    dev = q.device
    sdt = _lib.code_dtype(lib.mlstm_b200_chunkwise_state_dtype(S, DHQK, DHHV, L, dt, im))
    h = torch.empty((B, NH, S, DHHV), dtype=q.dtype, device=dev)
    n_out = torch.empty((B, NH, S), dtype=torch.float32, device=dev)
    m_out = torch.empty((B, NH, S), dtype=torch.float32, device=dev)
    c_states = torch.empty((B, NH, NC + 1, DHQK, DHHV), dtype=sdt, device=dev)
    # mLSTMsig without normaliser never writes n: the buffers are then zero-filled, otherwise fully overwritten
    n_alloc = torch.zeros if variant == _lib.SIG_NONORM else torch.empty
    n_states = n_alloc((B, NH, NC + 1, DHQK), dtype=torch.float32, device=dev)
    m_states = torch.empty((B, NH, NC + 1), dtype=torch.float32, device=dev)
    c_last = n_last = m_last = None
    if want_last:
        c_last = torch.empty((B, NH, DHQK, DHHV), dtype=torch.float32, device=dev)
        n_last = n_alloc((B, NH, DHQK), dtype=torch.float32, device=dev)
        m_last = torch.empty((B, NH, 1), dtype=torch.float32, device=dev)
    ws_bytes = lib.mlstm_b200_chunkwise_workspace_bytes(B, NH, S, DHQK, DHHV, L, dt, variant, im, 0)
    ws = torch.empty((max(ws_bytes, 256),), dtype=torch.uint8, device=dev)
    with torch.cuda.device(dev):
        rc = lib.mlstm_b200_chunkwise_fw(
            _lib.ptr(q), _lib.ptr(k), _lib.ptr(v), _lib.ptr(i), _lib.ptr(f),
            _lib.ptr(c0), _lib.ptr(n0), _lib.ptr(m0),
            _lib.ptr(h), _lib.ptr(n_out), _lib.ptr(m_out),
            _lib.ptr(c_states), _lib.ptr(n_states), _lib.ptr(m_states),
            _lib.ptr(c_last), _lib.ptr(n_last), _lib.ptr(m_last),
            _lib.ptr(ws), ws_bytes, B, NH, S, DHQK, DHHV, L, dt, gdt, variant, im, float(eps),
            _lib.stream_handle(dev))
    _lib.check(rc, "mlstm_b200_chunkwise_fw")
    return dict(H=h, n_out=n_out, m_out=m_out, C_states=c_states, n_states=n_states, m_states=m_states,
                C_last=c_last, n_last=n_last, m_last=m_last, workspace=ws)


def chunkwise_states_raw(k, v, i, f, c_initial=None, m_initial=None, *, chunk_size: int, variant: int,
                         impl: str = "auto", fw_workspace=None):
    """Per-chunk C states (B, NH, NC+1, DHQK, DHHV) alone: the forward's recurrence re-run for a backward whose
    forward did not keep them.  With `fw_workspace` (as returned by chunkwise_fw_raw for the same inputs) the gate
    pre-pass is not repeated."""
    _lib.require_cuda(k, v, i, f)
    lib = _lib.load()
    B, NH, S, DHQK = k.shape
    DHHV = v.shape[-1]
    L = chunk_size
    dt, gdt, im = _lib.dtype_code(k.dtype), _lib.dtype_code(i.dtype), _lib.IMPL[impl]
    if i.dtype != f.dtype:
        f = f.to(i.dtype)
    k, v, i, f = (t.contiguous() for t in (k, v, i, f))
    c0 = _f32c(c_initial)
    m0 = None if m_initial is None else _f32c(m_initial).reshape(B, NH)
    dev = k.device
    sdt = _lib.code_dtype(lib.mlstm_b200_chunkwise_state_dtype(S, DHQK, DHHV, L, dt, im))
    c_states = torch.empty((B, NH, -(-S // L) + 1, DHQK, DHHV), dtype=sdt, device=dev)
    ws, ws_bytes = None, 0
    if fw_workspace is None:
        ws_bytes = lib.mlstm_b200_chunkwise_workspace_bytes(B, NH, S, DHQK, DHHV, L, dt, variant, im, 2)
        ws = torch.empty((max(ws_bytes, 256),), dtype=torch.uint8, device=dev)
    with torch.cuda.device(dev):
        rc = lib.mlstm_b200_chunkwise_states(
            _lib.ptr(k), _lib.ptr(v), _lib.ptr(i), _lib.ptr(f), _lib.ptr(c0), _lib.ptr(m0), _lib.ptr(c_states),
            _lib.ptr(fw_workspace), 0 if fw_workspace is None else fw_workspace.numel(), _lib.ptr(ws), ws_bytes,
            B, NH, S, DHQK, DHHV, L, dt, gdt, variant, im, _lib.stream_handle(dev))
    _lib.check(rc, "mlstm_b200_chunkwise_states")
    return c_states


def chunkwise_bw_raw(q, k, v, i, f, m_initial, c_states, n_out, dh, dc_last=None, *, chunk_size: int, eps: float,
                     variant: int, impl: str = "auto", want_dc_initial: bool = False, m_out=None, fw_workspace=None,
                     recompute_c_initial=None):
    """Run the backward kernels.  Returns (dq, dk, dv, di, df, dc_initial).  With `m_out` and `fw_workspace` (both
    as returned by chunkwise_fw_raw for the same inputs) the gate pre-pass is not repeated.  With c_states = None
    (needs fw_workspace) the per-chunk states are recomputed inside the call, from `recompute_c_initial`."""
    _lib.require_cuda(q, k, v, i, f, dh)
    lib = _lib.load()
    B, NH, S, DHQK = q.shape
    DHHV = v.shape[-1]
    L = chunk_size
    dt, gdt, im = _lib.dtype_code(q.dtype), _lib.dtype_code(i.dtype), _lib.IMPL[impl]
    if i.dtype != f.dtype:
        f = f.to(i.dtype)
    q, k, v, i, f = (t.contiguous() for t in (q, k, v, i, f))
    dh = dh.to(q.dtype).contiguous()
    dcl = _f32c(dc_last)
    m0 = None if m_initial is None else _f32c(m_initial).reshape(B, NH)
    dev = q.device
    dq = torch.empty_like(q)
    dk = torch.empty_like(k)
    dv = torch.empty_like(v)
    di = torch.empty((B, NH, S), dtype=torch.float32, device=dev)
    df = torch.empty((B, NH, S), dtype=torch.float32, device=dev)
    dc0 = torch.empty((B, NH, DHQK, DHHV), dtype=torch.float32, device=dev) if want_dc_initial else None
    ws_bytes = lib.mlstm_b200_chunkwise_workspace_bytes(B, NH, S, DHQK, DHHV, L, dt, variant, im, 1)
    ws = torch.empty((max(ws_bytes, 256),), dtype=torch.uint8, device=dev)
    with torch.cuda.device(dev):
        if c_states is None:
            if fw_workspace is None:
                raise ValueError("recomputing the states inside the backward needs the forward's workspace")
            sdt = _lib.code_dtype(lib.mlstm_b200_chunkwise_state_dtype(S, DHQK, DHHV, L, dt, im))
            c_states = torch.empty((B, NH, -(-S // L) + 1, DHQK, DHHV), dtype=sdt, device=dev)
            c0 = _f32c(recompute_c_initial)
            rc = lib.mlstm_b200_chunkwise_bw_recompute(
                _lib.ptr(q), _lib.ptr(k), _lib.ptr(v), _lib.ptr(i), _lib.ptr(f),
                _lib.ptr(m0), _lib.ptr(c0), _lib.ptr(c_states), _lib.ptr(n_out), _lib.ptr(m_out),
                _lib.ptr(fw_workspace), fw_workspace.numel(), _lib.ptr(dh), _lib.ptr(dcl),
                _lib.ptr(dq), _lib.ptr(dk), _lib.ptr(dv), _lib.ptr(di), _lib.ptr(df), _lib.ptr(dc0),
                _lib.ptr(ws), ws_bytes, B, NH, S, DHQK, DHHV, L, dt, gdt, variant, im, float(eps),
                _lib.stream_handle(dev))
        elif fw_workspace is not None and m_out is not None:
            rc = lib.mlstm_b200_chunkwise_bw_cached(
                _lib.ptr(q), _lib.ptr(k), _lib.ptr(v), _lib.ptr(i), _lib.ptr(f),
                _lib.ptr(m0), _lib.ptr(c_states), _lib.ptr(n_out), _lib.ptr(m_out), _lib.ptr(fw_workspace),
                fw_workspace.numel(), _lib.ptr(dh), _lib.ptr(dcl),
                _lib.ptr(dq), _lib.ptr(dk), _lib.ptr(dv), _lib.ptr(di), _lib.ptr(df), _lib.ptr(dc0),
                _lib.ptr(ws), ws_bytes, B, NH, S, DHQK, DHHV, L, dt, gdt, variant, im, float(eps),
                _lib.stream_handle(dev))
        else:
            rc = lib.mlstm_b200_chunkwise_bw(
                _lib.ptr(q), _lib.ptr(k), _lib.ptr(v), _lib.ptr(i), _lib.ptr(f),
                _lib.ptr(m0), _lib.ptr(c_states), _lib.ptr(n_out), _lib.ptr(dh), _lib.ptr(dcl),
                _lib.ptr(dq), _lib.ptr(dk), _lib.ptr(dv), _lib.ptr(di), _lib.ptr(df), _lib.ptr(dc0),
                _lib.ptr(ws), ws_bytes, B, NH, S, DHQK, DHHV, L, dt, gdt, variant, im, float(eps),
                _lib.stream_handle(dev))
    _lib.check(rc, "mlstm_b200_chunkwise_bw")
    return dq, dk, dv, di, df, dc0


def _make_fwbw(autocast_kernel_dtype: torch.dtype, variant: int):
    class _mlstm_chunkwise_fwbw(torch.autograd.Function):
        @staticmethod
        @custom_fwd(device_type="cuda", cast_inputs=autocast_kernel_dtype)
        def forward(ctx, q, k, v, i, f, c_initial, n_initial, m_initial, return_last_states, eps, chunk_size, impl,
                    recompute_states_in_bw):
            B, NH, S, DHQK = q.shape
            L = resolve_chunk_size(q, v, chunk_size, impl)
            out = chunkwise_fw_raw(q, k, v, i, f, c_initial, n_initial, m_initial, chunk_size=L, eps=eps,
                                   variant=variant, impl=impl, want_last=return_last_states)
            # The forward's gate vectors (its scratch buffer and m_out) are kept for the backward: 24 B per token.
            # The per-chunk C states (2 * DHQK * DHHV / L bytes per token on the tcgen05 path) are kept only when
            # the caller asks for it; otherwise the backward runs the recurrence again, as the reference does
            # (mlstm_kernels/torch/chunkwise/triton_xl_chunk/fwbw.py:88-115).
            kept = None if recompute_states_in_bw else out["C_states"]
            ctx.save_for_backward(q, k, v, i, f, c_initial if recompute_states_in_bw else None, m_initial, kept,
                                  out["n_out"], out["m_out"], out["workspace"])
            ctx.cfg = (L, eps, impl, c_initial is not None, n_initial is not None, m_initial is not None,
                       None if c_initial is None else c_initial.dtype,
                       None if n_initial is None else n_initial.dtype)
            ctx.mark_non_differentiable(out["n_out"], out["m_out"])
            if return_last_states:
                return out["H"], out["C_last"], out["n_last"], out["m_last"]
            return out["H"], None, None, None

        @staticmethod
        @custom_bwd(device_type="cuda")
        def backward(ctx, dH, dC_last, dN_last, dM_last):
            q, k, v, i, f, c_initial, m_initial, c_states, n_out, m_out, fw_ws = ctx.saved_tensors
            L, eps, impl, has_c0, has_n0, has_m0, c0_dtype, n0_dtype = ctx.cfg
            # c_states is None: the forward did not keep them; the call runs the recurrence again in front of its own
            # chains of launches
            dq, dk, dv, di, df, dc0 = chunkwise_bw_raw(
                q, k, v, i, f, m_initial, c_states, n_out, dH, dC_last, chunk_size=L, eps=eps, variant=variant,
                impl=impl, want_dc_initial=has_c0, m_out=m_out, fw_workspace=fw_ws, recompute_c_initial=c_initial)
            B, NH, S, DHQK = q.shape
            dn0 = torch.zeros((B, NH, DHQK), dtype=n0_dtype, device=q.device) if has_n0 else None
            dm0 = torch.zeros_like(m_initial) if has_m0 else None
            if dc0 is not None:
                dc0 = dc0.to(c0_dtype)
            if _CHECK_STATUS and _lib.device_status() != 0:
                raise RuntimeError("mlstm_kernels_b200: a bounded wait of the tcgen05 kernels ran out; results invalid")
            return (dq, dk, dv, di.to(i.dtype), df.to(f.dtype), dc0, dn0, dm0, None, None, None, None, None)

    return _mlstm_chunkwise_fwbw


_FWBW = {}


def _get_fwbw(autocast_kernel_dtype: torch.dtype, variant: int):
    if autocast_kernel_dtype not in (torch.float32, torch.float16, torch.bfloat16):
        raise ValueError(f"Unsupported kernel dtype {autocast_kernel_dtype}.")
    key = (autocast_kernel_dtype, variant)
    if key not in _FWBW:
        _FWBW[key] = _make_fwbw(autocast_kernel_dtype, variant)
    return _FWBW[key]


def mlstm_chunkwise__b200_xl_chunk(
    q: torch.Tensor,  # (B, NH, S, DHQK)
    k: torch.Tensor,  # (B, NH, S, DHQK)
    v: torch.Tensor,  # (B, NH, S, DHHV)
    i: torch.Tensor,  # (B, NH, S)
    f: torch.Tensor,  # (B, NH, S)
    c_initial: torch.Tensor = None,  # (B, NH, DHQK, DHHV)
    n_initial: torch.Tensor = None,  # (B, NH, DHQK)
    m_initial: torch.Tensor = None,  # (B, NH, 1)
    return_last_states: bool = False,
    eps: float = 1e-6,
    chunk_size: int = 128,
    chunk_size_inter: int | None = None,
    chunk_size_intra: int | None = None,
    siz_b_L_parallel: int | None = None,
    siz_b_L_loop: int | None = None,
    siz_b_DH_parallel: int | None = None,
    siz_b_DH_loop: int | None = None,
    num_warps_intra: int | None = None,
    num_warps_inter: int | None = None,
    num_stages_intra: int | None = None,
    num_stages_inter: int | None = None,
    recompute_states_in_bw: bool = True,
    autocast_kernel_dtype: torch.dtype = torch.float32,
    impl: str = "auto",
) -> torch.Tensor | tuple[torch.Tensor, tuple[torch.Tensor, torch.Tensor, torch.Tensor]]:
    """mLSTMexp chunkwise forward with autograd.  Returns H, or (H, (C_last, n_last, m_last)) with f32
    states when return_last_states is set.  `recompute_states_in_bw` has the reference's meaning (and default):
    True keeps only q, k, v, i, f and the per-token gate vectors between forward and backward and runs the
    inter-chunk recurrence again in the backward; False keeps the per-chunk C states (faster backward, more
    memory).  Tile / warp / stage arguments and chunk_size_inter / chunk_size_intra are Triton tuning knobs of
    the reference and have no meaning here."""
    if torch.compiler.is_compiling():   # a tracer is watching: go through the custom operators
        h, c_last, n_last, m_last = _ops.chunkwise_traced(
            q, k, v, i, f, c_initial, n_initial, m_initial, return_last_states, eps, chunk_size, impl,
            bool(recompute_states_in_bw), autocast_kernel_dtype, _lib.EXP)
    else:
        fn = _get_fwbw(autocast_kernel_dtype, _lib.EXP)
        h, c_last, n_last, m_last = fn.apply(q, k, v, i, f, c_initial, n_initial, m_initial, return_last_states,
                                             eps, chunk_size, impl, bool(recompute_states_in_bw))
    if return_last_states:
        return h, (c_last, n_last, m_last)
    return h


def mlstm_siging_chunkwise__b200_xl_chunk(
    q: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    i: torch.Tensor,
    f: torch.Tensor,
    c_initial: torch.Tensor = None,
    n_initial: torch.Tensor = None,
    m_initial: torch.Tensor = None,  # unused: placeholder to match the mLSTMexp interface
    return_last_states: bool = False,
    eps: float = 1e-6,
    normalize: bool = True,
    chunk_size: int = 128,
    chunk_size_inter: int | None = None,
    chunk_size_intra: int | None = None,
    siz_b_L_parallel: int | None = None,
    siz_b_L_loop: int | None = None,
    siz_b_DH_parallel: int | None = None,
    siz_b_DH_loop: int | None = None,
    num_warps_intra: int | None = None,
    num_warps_inter: int | None = None,
    num_stages_intra: int | None = None,
    num_stages_inter: int | None = None,
    recompute_states_in_bw: bool = True,
    autocast_kernel_dtype: torch.dtype = torch.float32,
    impl: str = "auto",
) -> torch.Tensor | tuple[torch.Tensor, tuple[torch.Tensor, torch.Tensor]]:
    """mLSTMsig (sigmoid input gate) chunkwise forward with autograd.  Returns H, or
    (H, (C_last, n_last)) when return_last_states is set."""
    variant = _lib.SIG if normalize else _lib.SIG_NONORM
    if torch.compiler.is_compiling():   # a tracer is watching: go through the custom operators
        h, c_last, n_last, _ = _ops.chunkwise_traced(
            q, k, v, i, f, c_initial, n_initial, None, return_last_states, eps, chunk_size, impl,
            bool(recompute_states_in_bw), autocast_kernel_dtype, variant)
    else:
        fn = _get_fwbw(autocast_kernel_dtype, variant)
        h, c_last, n_last, _ = fn.apply(q, k, v, i, f, c_initial, n_initial, None, return_last_states, eps,
                                        chunk_size, impl, bool(recompute_states_in_bw))
    if return_last_states:
        return h, (c_last, n_last)
    return h
