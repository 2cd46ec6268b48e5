"""Host-side logic of the multi-GPU modes, run as two gloo ranks on CPU.  The CUDA entry points are
replaced by the numpy oracle here (the kernels themselves are covered by the GPU tests); what is tested
is the partitioning, the point-to-point state hand-off along the chain and the combine arithmetic."""

import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from inputs import make_chunkwise_inputs, max_rel_err
from mlstm_kernels_b200 import sharding
from oracle import mlstm_oracle as O


def test_shard_range_partitions_units():
    for total in (1, 7, 64, 128, 2048):
        for world in (1, 2, 4, 8):
            spans = [sharding.shard_range(total, world, r) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == total
            assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
            sizes = [b - a for a, b in spans]
            assert max(sizes) - min(sizes) <= 1
    with pytest.raises(ValueError):
        sharding.shard_range(8, 2, 2)


def test_shard_batch_heads_slices_units():
    q = torch.arange(2 * 4 * 3 * 5, dtype=torch.float32).reshape(2, 4, 3, 5)
    i = torch.arange(2 * 4 * 3, dtype=torch.float32).reshape(2, 4, 3)
    parts = [sharding.shard_batch_heads([q, i], 4, r) for r in range(4)]
    assert torch.equal(torch.cat([p[0] for p in parts], 1).reshape(2, 4, 3, 5), q)
    assert torch.equal(torch.cat([p[1] for p in parts], 1).reshape(2, 4, 3), i)


# ---- oracle-backed stand-ins for the CUDA entry points --------------------------------------------
def _np(t):
    return None if t is None else t.detach().double().numpy()


def fake_segment_summary(k, v, i, f, *, chunk_size, variant, impl="auto"):
    B, NH, S, DHQK = k.shape
    siging = variant != 0
    fw = O.chunkwise_fw(np.zeros_like(_np(k)), _np(k), _np(v), _np(i), _np(f), None, None,
                        None if siging else np.full((B, NH, 1), -np.inf), chunk_size=chunk_size, siging=siging)
    g = O.logsigmoid(_np(f)).sum(-1)
    t = lambda x: torch.from_numpy(np.ascontiguousarray(x)).float()  # noqa: E731
    return t(fw["C_last"]), t(fw["n_last"]), t(fw["m_last"]), t(g)


def fake_state_combine(state_in, summary, *, variant):
    c_in, n_in, m_in = (x.double() for x in state_in)
    c_loc, n_loc, m_loc, g = (x.double() for x in summary)
    if variant == 0:
        m_out = torch.maximum(g[..., None] + m_in, m_loc)
        a, b = torch.exp(g[..., None] + m_in - m_out), torch.exp(m_loc - m_out)
    else:
        m_out = torch.zeros_like(m_loc)
        a, b = torch.exp(g[..., None]), torch.ones_like(m_loc)
    return ((a[..., None] * c_in + b[..., None] * c_loc).float(), (a * n_in + b * n_loc).float(), m_out.float())


def fake_segment_forward_saved(q, k, v, i, f, state_in, *, chunk_size, eps, variant, impl):
    siging = variant != 0
    fw = O.chunkwise_fw(_np(q), _np(k), _np(v), _np(i), _np(f), _np(state_in[0]), _np(state_in[1]),
                        None if siging else _np(state_in[2]), chunk_size=chunk_size, eps=eps, siging=siging,
                        normalize=variant != 2)
    t = lambda x: torch.from_numpy(np.ascontiguousarray(x)).float()  # noqa: E731
    fw.update(_k=_np(k), _v=_np(v), _i=_np(i), _f=_np(f))
    return t(fw["H"]), (t(fw["C_last"]), t(fw["n_last"]), t(fw["m_last"])), dict(fw=fw)


def fake_segment_backward(q, k, v, i, f, saved, dh, dc_last, *, chunk_size, eps, variant, impl):
    siging = variant != 0
    bw = O.chunkwise_bw(_np(q), _np(k), _np(v), _np(i), _np(f), _np(dh), saved["fw"], _np(dc_last), True,
                        chunk_size=chunk_size, eps=eps, siging=siging, normalize=variant != 2)
    t = lambda x: torch.from_numpy(np.ascontiguousarray(x)).float()  # noqa: E731
    return t(bw["dQ"]), t(bw["dK"]), t(bw["dV"]), t(bw["dI"]), t(bw["dF"]), t(bw["dC_initial"])


def fake_segment_dc_summary(q, dh, saved, *, chunk_size, eps, variant, impl="auto"):
    siging = variant != 0
    fw = saved["fw"]
    # only the state-gradient recurrence matters here: it reads q, dh and the forward's gates and normaliser
    bw = O.chunkwise_bw(_np(q), fw["_k"], fw["_v"], fw["_i"], fw["_f"], _np(dh), fw, None, True,
                        chunk_size=chunk_size, eps=eps, siging=siging, normalize=variant != 2)
    return torch.from_numpy(np.ascontiguousarray(bw["dC_initial"])).float()


CASE = dict(seed=17, B=1, NH=2, S=256, DHQK=16, DHHV=32, f_offset=1.0)


def _initial_state():
    rng = np.random.default_rng(99)
    B, NH, DHQK, DHHV = CASE["B"], CASE["NH"], CASE["DHQK"], CASE["DHHV"]
    return (0.1 * rng.standard_normal((B, NH, DHQK, DHHV)).astype(np.float32),
            np.abs(rng.standard_normal((B, NH, DHQK))).astype(np.float32),
            rng.standard_normal((B, NH, 1)).astype(np.float32))


def _worker(rank, world, port, mode, siging, out_dir, with_initial=False):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    sharding.segment_summary = fake_segment_summary
    sharding.state_combine = fake_state_combine
    sharding._segment_forward_saved = fake_segment_forward_saved
    sharding._segment_backward = fake_segment_backward
    sharding.segment_dc_summary = fake_segment_dc_summary
    inp = make_chunkwise_inputs(CASE)
    seg = CASE["S"] // world
    sl = slice(rank * seg, (rank + 1) * seg)
    q, k, v, i, f = (torch.from_numpy(inp[n][:, :, sl].copy()).requires_grad_(True) for n in "qkvif")
    c0 = n0 = m0 = None
    if with_initial:   # the state entering the whole sequence: only rank 0's copy is used
        c0, n0, m0 = (torch.from_numpy(x) for x in _initial_state())
        if rank != 0:
            c0, n0, m0 = torch.full_like(c0, 7.0), torch.full_like(n0, 7.0), torch.full_like(m0, 7.0)
    h, last = sharding.mlstm_chunkwise_sequence_parallel(q, k, v, i, f, c0, n0, None if siging else m0,
                                                         return_last_states=True, chunk_size=32,
                                                         siging=siging, mode=mode)
    (h * torch.from_numpy(inp["dH"][:, :, sl].copy())).sum().backward()   # chain of messages from the last rank back
    np.savez(os.path.join(out_dir, f"r{rank}.npz"), h=h.detach().numpy(),
             **{f"s{j}": t.numpy() for j, t in enumerate(last)},
             **{"d" + n: t.grad.numpy() for n, t in zip("qkvif", (q, k, v, i, f))})
    dist.destroy_process_group()


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


@pytest.mark.parametrize("mode,world", [("gather", 2), ("scan", 2), ("chain", 2), ("scan", 4), ("gather", 4)])
@pytest.mark.parametrize("siging", [False, True])
def test_sequence_parallel_gloo_ranks(tmp_path, mode, world, siging):
    mp.spawn(_worker, args=(world, _free_port(), mode, siging, str(tmp_path)), nprocs=world, join=True)
    inp = make_chunkwise_inputs(CASE)
    full, full_bw = O.chunkwise_fwbw(inp["q"], inp["k"], inp["v"], inp["i"], inp["f"], inp["dH"], chunk_size=32,
                                     siging=siging)
    outs = [dict(np.load(tmp_path / f"r{r}.npz")) for r in range(world)]
    h = np.concatenate([o["h"] for o in outs], axis=2)
    assert max_rel_err(h, full["H"]) < 1e-5
    for o in outs:  # the final state is broadcast to every rank
        assert max_rel_err(o["s0"], full["C_last"]) < 1e-5
        assert max_rel_err(o["s1"], full["n_last"]) < 1e-5
        if not siging:
            assert max_rel_err(o["s2"], full["m_last"]) < 1e-6
    # gradients of the whole sequence, assembled from the ranks' segments
    for n, key in (("q", "dQ"), ("k", "dK"), ("v", "dV"), ("i", "dI"), ("f", "dF")):
        got = np.concatenate([o["d" + n] for o in outs], axis=2)
        assert max_rel_err(got, full_bw[key]) < 1e-5, key


@pytest.mark.parametrize("mode", ["gather", "scan", "chain"])
@pytest.mark.parametrize("siging", [False, True])
def test_sequence_parallel_with_an_initial_state(tmp_path, mode, siging):
    """The state entering the whole sequence is rank 0's argument (the other ranks pass garbage here): every mode has
    to carry it through the hand-off to every later segment."""
    world = 4 if mode == "gather" else 2
    mp.spawn(_worker, args=(world, _free_port(), mode, siging, str(tmp_path), True), nprocs=world, join=True)
    inp = make_chunkwise_inputs(CASE)
    c0, n0, m0 = _initial_state()
    full, full_bw = O.chunkwise_fwbw(*(inp[n] for n in ("q", "k", "v", "i", "f", "dH")), c_initial=c0,
                                     n_initial=n0, m_initial=None if siging else m0, chunk_size=32, siging=siging)
    outs = [dict(np.load(tmp_path / f"r{r}.npz")) for r in range(world)]
    assert max_rel_err(np.concatenate([o["h"] for o in outs], axis=2), full["H"]) < 1e-5
    for o in outs:
        assert max_rel_err(o["s0"], full["C_last"]) < 1e-5
    for n, key in (("q", "dQ"), ("k", "dK"), ("v", "dV"), ("i", "dI"), ("f", "dF")):
        assert max_rel_err(np.concatenate([o["d" + n] for o in outs], axis=2), full_bw[key]) < 1e-5, key
