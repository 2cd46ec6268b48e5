"""Multi-GPU use of the chunkwise kernels: one process per GPU, `torch.distributed` for the plumbing.

Two modes (the reference itself is single-device; both build on its state-passing contract,
c_initial / n_initial / m_initial in, last states out: mlstm_kernels/torch/kernel_wrappers.py:109-151):

* batch x heads sharding: every (batch, head) pair is an independent unit in all kernels, so the units
  are split contiguously over the ranks and no data-path collective is needed (`shard_range`,
  `shard_batch_heads`).
* sequence-parallel prefill of one long sequence (`mlstm_chunkwise_sequence_parallel`): rank r holds the
  r-th contiguous segment of the sequence.  "scan" mode: (1) all ranks compute, concurrently, the state
  their segment produces from the empty state; (2) the boundary state travels along the chain
  rank 0 -> 1 -> ... with one point-to-point message per boundary ((C, n, m) packed into one buffer; NCCL
  send/recv, i.e. NVLink between GPUs of a node), each rank folding its summary onto the incoming state; (3) all ranks run the full
  forward of their segment, concurrently, from the true incoming state.  "chain" mode is the plain
  serial hand-off (segment r starts when r-1 has finished its recurrence).  Both reproduce the
  single-GPU (C, n, m) path.
  The call is differentiable.  "chain" mode runs the chain the other way: rank r receives, from rank r+1, the
  gradient of the state it handed over and the sum of (q . dq - k . dk) over all later tokens of each head
  (the forget-gate gradient of a token is sigmoid(-f) times that sum over all tokens from it to the end of the
  WHOLE sequence: mlstm_kernels/torch/chunkwise/triton_xl_chunk/chunkwise_gates.py:75-95), runs the backward of its
  segment, and passes both on to rank r-1.
  "scan" mode keeps the segment backwards concurrent as well.  The state-gradient recurrence is linear in the
  gradient that enters it on the right, dC_left = a dC_right + dC_own with a = exp(G + m_in - m_out) per head
  (exp(G) for the sigmoid input gate), so (1) all ranks compute dC_own (`segment_dc_summary`: the light recurrence
  only, from a zero gradient), (2) only the (B, NH, DHQK, DHHV) boundary gradient travels along the chain, one
  multiply-add per hop, (3) all ranks run the full backward of their segment from the true dC_right.  The sum over
  all later tokens needs no message: summed from a chunk boundary to the end of the sequence,
  q . dq - k . dk = <C, dC> at that boundary, so it is <C_last, dC_right> of the rank's own segment.
  "gather" mode (what "auto" picks from three ranks on; with two ranks it picks "scan") replaces both chains by one
  all-gather each: every rank receives all segment summaries
  and folds those of the ranks before it itself, in rank order (the same arithmetic in the same order as the chain,
  so the same bits); in the backward every rank receives all (dC_own, a) pairs and folds those of the ranks after it.
  The hops of a chain are serial - each costs a message latency plus the launches around it, seven of them on eight
  GPUs - while the folds are a few small kernels on data that one collective over NVSwitch has already delivered.
"""

from __future__ import annotations

import torch
import torch.distributed as dist

from . import _lib
from .chunkwise import chunkwise_bw_raw, chunkwise_fw_raw, resolve_chunk_size


def shard_range(total: int, world: int, rank: int) -> tuple[int, int]:
    """Contiguous [start, stop) of `total` units owned by `rank`; sizes differ by at most one."""
    if world <= 0 or not (0 <= rank < world):
        raise ValueError(f"bad rank {rank} for world size {world}")
    base, rem = divmod(total, world)
    start = rank * base + min(rank, rem)
    return start, start + base + (1 if rank < rem else 0)


def shard_batch_heads(tensors, world: int, rank: int):
    """Slice the (B, NH, ...) tensors to this rank's share of the B*NH independent units.
    Returns tensors of shape (1, units, ...) (views when the inputs are contiguous)."""
    B, NH = tensors[0].shape[:2]
    start, stop = shard_range(B * NH, world, rank)
    return [t.reshape(1, B * NH, *t.shape[2:])[:, start:stop] for t in tensors]


def _variant(siging: bool, normalize: bool) -> int:
    return _lib.EXP if not siging else (_lib.SIG if normalize else _lib.SIG_NONORM)


def segment_summary(k, v, i, f, *, chunk_size: int, variant: int, impl: str = "auto"):
    """State (C, n, m) and total log forget gate G that one segment produces from the empty state."""
    _lib.require_cuda(k, v, i, f)
    lib = _lib.load()
    B, NH, S, DHQK = k.shape
    DHHV = v.shape[-1]
    dt, gdt, im = _lib.dtype_code(k.dtype), _lib.dtype_code(i.dtype), _lib.IMPL[impl]
    k, v, i, f = (t.contiguous() for t in (k, v, i, f.to(i.dtype)))
    dev = k.device
    c = torch.empty((B, NH, DHQK, DHHV), dtype=torch.float32, device=dev)
    n = torch.zeros((B, NH, DHQK), dtype=torch.float32, device=dev)
    m = torch.empty((B, NH, 1), dtype=torch.float32, device=dev)
    g = torch.empty((B, NH), dtype=torch.float32, device=dev)
    ws_bytes = lib.mlstm_b200_chunkwise_workspace_bytes(B, NH, S, DHQK, DHHV, chunk_size, dt, variant, im, 2)
    ws = torch.empty((max(ws_bytes, 256),), dtype=torch.uint8, device=dev)
    with torch.cuda.device(dev):
        rc = lib.mlstm_b200_chunkwise_summary(
            _lib.ptr(k), _lib.ptr(v), _lib.ptr(i), _lib.ptr(f), _lib.ptr(c),
            None if variant == _lib.SIG_NONORM else _lib.ptr(n), _lib.ptr(m), _lib.ptr(g), _lib.ptr(ws), ws_bytes,
            B, NH, S, DHQK, DHHV, chunk_size, dt, gdt, variant, im, _lib.stream_handle(dev))
    _lib.check(rc, "mlstm_b200_chunkwise_summary")
    return c, n, m, g


def state_combine(state_in, summary, *, variant: int):
    """Fold a segment summary (C_loc, n_loc, m_loc, G) onto the state (C, n, m) entering the segment."""
    c_in, n_in, m_in = state_in
    c_loc, n_loc, m_loc, g = summary
    lib = _lib.load()
    B, NH, DHQK, DHHV = c_loc.shape
    dev = c_loc.device
    c_out, n_out, m_out = torch.empty_like(c_loc), torch.zeros_like(n_loc), torch.zeros_like(m_loc)
    f32 = lambda t: None if t is None else t.to(torch.float32).contiguous()  # noqa: E731
    c_in, n_in, m_in = f32(c_in), f32(n_in), f32(m_in)
    with torch.cuda.device(dev):
        rc = lib.mlstm_b200_state_combine(
            _lib.ptr(c_in), _lib.ptr(n_in), _lib.ptr(m_in), _lib.ptr(c_loc), _lib.ptr(n_loc), _lib.ptr(m_loc),
            _lib.ptr(g), _lib.ptr(c_out), None if variant == _lib.SIG_NONORM else _lib.ptr(n_out), _lib.ptr(m_out),
            B, NH, DHQK, DHHV, variant, _lib.stream_handle(dev))
    _lib.check(rc, "mlstm_b200_state_combine")
    return c_out, n_out, m_out


def _segment_forward_saved(q, k, v, i, f, state_in, *, chunk_size, eps, variant, impl):
    """Forward of one segment that also returns what its backward needs."""
    c0, n0, m0 = state_in
    out = chunkwise_fw_raw(q, k, v, i, f, c0, n0, m0 if variant == _lib.EXP else None, chunk_size=chunk_size,
                           eps=eps, variant=variant, impl=impl, want_last=True)
    saved = dict(m_initial=m0 if variant == _lib.EXP else None, c_states=out["C_states"], n_out=out["n_out"],
                 m_out=out["m_out"], workspace=out["workspace"])
    return out["H"], (out["C_last"], out["n_last"], out["m_last"]), saved


def _segment_backward(q, k, v, i, f, saved, dh, dc_last, *, chunk_size, eps, variant, impl):
    """Backward of one segment: (dq, dk, dv, di, df, gradient of the state the segment received)."""
    return chunkwise_bw_raw(q, k, v, i, f, saved["m_initial"], saved["c_states"], saved["n_out"], dh, dc_last,
                            chunk_size=chunk_size, eps=eps, variant=variant, impl=impl, want_dc_initial=True,
                            m_out=saved["m_out"], fw_workspace=saved["workspace"])


def segment_dc_summary(q, dh, saved, *, chunk_size, eps, variant, impl="auto"):
    """The segment's own contribution to the gradient of the state that entered it: its state-gradient recurrence
    started from a zero gradient on the right.  (B, NH, DHQK, DHHV) f32.  No per-chunk states are written."""
    _lib.require_cuda(q, dh)
    lib = _lib.load()
    B, NH, S, DHQK = q.shape
    DHHV = dh.shape[-1]
    dt, im = _lib.dtype_code(q.dtype), _lib.IMPL[impl]
    q, dh = q.contiguous(), dh.to(q.dtype).contiguous()
    dev = q.device
    dc = torch.empty((B, NH, DHQK, DHHV), dtype=torch.float32, device=dev)
    sp = -(-S // chunk_size) * chunk_size
    ws = torch.empty((max(B * NH * sp * 4 + 256, 256),), dtype=torch.uint8, device=dev)
    fw_ws = saved["workspace"]
    with torch.cuda.device(dev):
        rc = lib.mlstm_b200_chunkwise_dc_summary(
            _lib.ptr(q), _lib.ptr(dh), None if variant == _lib.SIG_NONORM else _lib.ptr(saved["n_out"]),
            _lib.ptr(fw_ws), fw_ws.numel(), _lib.ptr(dc), _lib.ptr(ws), ws.numel(),
            B, NH, S, DHQK, DHHV, chunk_size, dt, variant, im, eps, _lib.stream_handle(dev))
    _lib.check(rc, "mlstm_b200_chunkwise_dc_summary")
    return dc


def _segment_gate_sum(q, k, f, dq, dk, df_local):
    """Sum over the segment's tokens of (q . dq - k . dk), per (batch, head).
    The kernels form these sums in f32 from their f32 accumulators and return them inside the forget-gate gradient:
    df_local[t] = sigmoid(-f[t]) * (sum over tokens t' >= t of the segment), so token 0 carries the whole sum.  The sum
    of the rounded dq, dk outputs is not used unless sigmoid(-f[0]) underflows: q . dq and k . dk nearly cancel, and the
    rounding of bf16 outputs would dominate their difference."""
    s0 = torch.sigmoid(-f[..., 0].float())
    from_df = df_local[..., 0].float() / s0.clamp_min(1e-30)
    fallback = (q.float() * dq.float() - k.float() * dk.float()).sum(dim=(-1, -2))
    return torch.where(s0 > 1e-30, from_df, fallback)


class _SequenceParallelFn(torch.autograd.Function):
    """Differentiable sequence-parallel forward; see the module docstring for the backward chain."""

    @staticmethod
    def forward(ctx, q, k, v, i, f, first_state, opts):
        group, ranks, rank, world = opts["group"], opts["ranks"], opts["rank"], opts["world"]
        L, eps, variant, impl, mode = opts["L"], opts["eps"], opts["variant"], opts["impl"], opts["mode"]
        prev_rank = ranks[rank - 1] if rank > 0 else None
        next_rank = ranks[rank + 1] if rank < world - 1 else None
        like = first_state
        if mode == "chain":
            state_in = first_state if rank == 0 else _recv_state(like, prev_rank, group)
            h, last, saved = _segment_forward_saved(q, k, v, i, f, state_in, chunk_size=L, eps=eps, variant=variant,
                                                    impl=impl)
            if next_rank is not None:
                _send_state(last, next_rank, group)
        else:
            summary = segment_summary(k, v, i, f, chunk_size=L, variant=variant, impl=impl)
            if mode == "gather":
                # rank 0 contributes the state at the end of its segment (the initial state of the whole sequence
                # folded in), every other rank its summary; rank r folds entries 1 .. r-1 onto entry 0
                mine = state_combine(first_state, summary, variant=variant) + (summary[3],) if rank == 0 else summary
                entries = _all_gather_packed(mine, world, group)
                state_in = first_state
                if rank > 0:
                    state_in = tuple(entries[0][:3])
                    for r in range(1, rank):
                        state_in = state_combine(state_in, entries[r], variant=variant)
                last = tuple(mine[:3]) if rank == 0 else state_combine(state_in, summary, variant=variant)
            else:
                state_in = first_state if rank == 0 else _recv_state(like, prev_rank, group)
                last = state_combine(state_in, summary, variant=variant)
                if next_rank is not None:
                    _send_state(last, next_rank, group)
            h, _, saved = _segment_forward_saved(q, k, v, i, f, state_in, chunk_size=L, eps=eps, variant=variant,
                                                 impl=impl)
            # per-head decay of a state gradient across the whole segment, and the state at its right end
            log_a = summary[3] + (state_in[2] - last[2]).reshape(summary[3].shape) if variant == _lib.EXP else summary[3]
            saved["decay"], saved["c_last"] = torch.exp(log_a), last[0]
        ctx.opts, ctx.saved = opts, saved
        ctx.save_for_backward(q, k, v, i, f)
        ctx.mark_non_differentiable(*last)
        return (h,) + tuple(last)

    @staticmethod
    def backward(ctx, dh, *_unused):
        q, k, v, i, f = ctx.saved_tensors
        opts = ctx.opts
        group, ranks, rank, world = opts["group"], opts["ranks"], opts["rank"], opts["world"]
        prev_rank = ranks[rank - 1] if rank > 0 else None
        next_rank = ranks[rank + 1] if rank < world - 1 else None
        B, NH, S, DHQK = q.shape
        DHHV = v.shape[-1]
        if opts["mode"] in ("scan", "gather"):
            kw = dict(chunk_size=opts["L"], eps=opts["eps"], variant=opts["variant"], impl=opts["impl"])
            dh = dh.contiguous()
            dc_right = None
            if opts["mode"] == "gather":
                # every rank receives every (dC_own, a) and folds those of the ranks after it, last rank first
                own = (segment_dc_summary(q, dh, ctx.saved, **kw) if rank > 0 else
                       torch.zeros((B, NH, DHQK, DHHV), dtype=torch.float32, device=q.device))
                entries = _all_gather_packed((own, ctx.saved["decay"]), world, group)
                for r in range(world - 1, rank, -1):
                    own_r, decay_r = entries[r]
                    dc_right = own_r if dc_right is None else own_r + decay_r[..., None, None] * dc_right
                dq, dk, dv, di, df, _ = _segment_backward(q, k, v, i, f, ctx.saved, dh, dc_right, **kw)
                if dc_right is not None:
                    tail = (ctx.saved["c_last"] * dc_right).sum(dim=(-1, -2))
                    df = df + torch.sigmoid(-f.float()) * tail[..., None]
                return dq, dk, dv, di.to(i.dtype), df.to(f.dtype), None, None
            if prev_rank is not None:   # rank 0 hands nothing on: it needs no summary
                dc_left = segment_dc_summary(q, dh, ctx.saved, **kw)
            if next_rank is not None:
                like = (torch.empty((B, NH, DHQK, DHHV), dtype=torch.float32, device=q.device),)
                (dc_right,) = _recv_state(like, next_rank, group)
                if prev_rank is not None:
                    dc_left = dc_left + ctx.saved["decay"][..., None, None] * dc_right
            if prev_rank is not None:
                _send_state((dc_left,), prev_rank, group)
            dq, dk, dv, di, df, _ = _segment_backward(q, k, v, i, f, ctx.saved, dh, dc_right, **kw)
            if dc_right is not None:
                tail = (ctx.saved["c_last"] * dc_right).sum(dim=(-1, -2))
                df = df + torch.sigmoid(-f.float()) * tail[..., None]
            return dq, dk, dv, di.to(i.dtype), df.to(f.dtype), None, None
        dc_last, tail = None, None
        if next_rank is not None:   # gradient of the state handed to rank r+1, and the sum over all later tokens
            like = (torch.empty((B, NH, DHQK, DHHV), dtype=torch.float32, device=q.device),
                    torch.empty((B, NH), dtype=torch.float32, device=q.device))
            dc_last, tail = _recv_state(like, next_rank, group)
        dq, dk, dv, di, df, dc0 = _segment_backward(q, k, v, i, f, ctx.saved, dh.contiguous(), dc_last,
                                                    chunk_size=opts["L"], eps=opts["eps"], variant=opts["variant"],
                                                    impl=opts["impl"])
        if prev_rank is not None:
            total = _segment_gate_sum(q, k, f, dq, dk, df)
            if tail is not None:
                total = total + tail
        if tail is not None:
            df = df + torch.sigmoid(-f.float()) * tail[..., None]
        if prev_rank is not None:
            _send_state((dc0, total), prev_rank, group)
        return dq, dk, dv, di.to(i.dtype), df.to(f.dtype), None, None


def _pack(tensors):
    """One flat f32 buffer holding the given tensors back to back (one message per hop instead of one per tensor)."""
    return torch.cat([t.reshape(-1).to(torch.float32) for t in tensors])


def _unpack(flat, like):
    out, off = [], 0
    for t in like:
        n = t.numel()
        out.append(flat[off:off + n].view(t.shape))
        off += n
    return tuple(out)


def _all_gather_packed(tensors, world, group):
    """All-gather of a tuple of tensors (packed into one f32 buffer per rank, one collective); returns, per rank of
    the group, the tuple of that rank's tensors."""
    flat = _pack(tensors)
    n = flat.numel()
    out = torch.empty(world * n, dtype=torch.float32, device=flat.device)
    dist.all_gather_into_tensor(out, flat, group=group)
    return [_unpack(out[r * n:(r + 1) * n], tensors) for r in range(world)]


def _send_state(state, dst, group):
    dist.send(_pack(state), dst=dst, group=group)


def _recv_state(like, src, group):
    flat = torch.empty(sum(t.numel() for t in like), dtype=torch.float32, device=like[0].device)
    dist.recv(flat, src=src, group=group)
    return _unpack(flat, like)


def mlstm_chunkwise_sequence_parallel(
    q: torch.Tensor,  # (B, NH, S_local, DHQK)  this rank's contiguous segment of the sequence
    k: torch.Tensor,
    v: torch.Tensor,  # (B, NH, S_local, DHHV)
    i: torch.Tensor,  # (B, NH, S_local)
    f: torch.Tensor,
    c_initial: torch.Tensor = None,  # state entering the WHOLE sequence (used by rank 0)
    n_initial: torch.Tensor = None,
    m_initial: torch.Tensor = None,
    return_last_states: bool = False,
    eps: float = 1e-6,
    chunk_size: int = 128,
    siging: bool = False,
    normalize: bool = True,
    mode: str = "auto",
    group=None,
    impl: str = "auto",
):
    """Forward (prefill) of one long sequence whose segments live on the ranks of `group`.
    Returns this rank's H (B, NH, S_local, DHHV) and, if requested, the state after the LAST segment
    (identical on every rank).  Ranks are ordered along the sequence: global rank order of the group.
    Differentiable with respect to q, k, v, i, f (every rank must then run the backward: it exchanges
    point-to-point messages from the last rank to the first)."""
    if mode not in ("auto", "gather", "scan", "chain"):
        raise ValueError(f"unknown mode {mode}")
    world = dist.get_world_size(group)
    if mode == "auto":   # a single hop needs no collective; from three ranks on the all-gather beats the serial hops
        mode = "scan" if world <= 2 else "gather"
    rank = dist.get_rank(group)
    variant = _variant(siging, normalize)
    B, NH, S, DHQK = q.shape
    DHHV = v.shape[-1]
    L = resolve_chunk_size(q, v, chunk_size, impl)
    dev = q.device
    ranks = dist.get_process_group_ranks(group) if group is not None else list(range(world))
    zeros = (torch.zeros((B, NH, DHQK, DHHV), dtype=torch.float32, device=dev),
             torch.zeros((B, NH, DHQK), dtype=torch.float32, device=dev),
             torch.zeros((B, NH, 1), dtype=torch.float32, device=dev))
    f32 = lambda t, z: z if t is None else t.to(torch.float32).contiguous()  # noqa: E731
    first_state = (f32(c_initial, zeros[0]), f32(n_initial, zeros[1]), f32(m_initial, zeros[2]))

    opts = dict(group=group, ranks=ranks, rank=rank, world=world, L=L, eps=eps, variant=variant, impl=impl, mode=mode)
    out = _SequenceParallelFn.apply(q, k, v, i, f, first_state, opts)
    h, last = out[0], out[1:]
    if not return_last_states:
        return h
    # one broadcast of the packed state, received into a buffer of its own: the state at the end of THIS rank's
    # segment stays as the backward saved it
    flat = _pack(last) if rank == world - 1 else torch.empty(sum(t.numel() for t in last), dtype=torch.float32,
                                                             device=dev)
    dist.broadcast(flat, src=ranks[world - 1], group=group)
    last = tuple(t.clone() for t in _unpack(flat, last))
    if siging:
        return h, (last[0], last[1])
    return h, last
