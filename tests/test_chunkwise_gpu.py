"""GPU parity tests of the chunkwise kernels: CUDA path (through the C ABI) vs the numpy oracle and
the committed golden vectors of the reference.  Error measure: max |x - ref| / max |ref|.

Stated tolerances
  f32 inputs : H, states 1e-4 ; gradients 1e-3
  bf16 inputs: H, gradients 2e-2 ; states 2e-2 (inputs of the oracle are rounded to bf16 first)
"""

import os

import numpy as np
import pytest
import torch

import mlstm_kernels_b200 as mk
from inputs import CASES, make_chunkwise_inputs, max_rel_err, subsample
from oracle import mlstm_oracle as O
from util_gpu import case_inputs, npy, run_cuda_fwbw, run_oracle_fwbw, to_dev

pytestmark = pytest.mark.gpu

GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
TOL_F32_FW, TOL_F32_BW, TOL_BF16 = 1e-4, 1e-3, 2e-2
FW_KEYS = ("H", "C_last", "n_last", "m_last")
BW_KEYS = ("dQ", "dK", "dV", "dI", "dF")


def compare(got, ref, tol_fw, tol_bw, keys_fw=FW_KEYS, stride=1):
    for key in keys_fw:
        if key in got and key in ref:
            assert max_rel_err(subsample(got[key], stride), subsample(np.asarray(ref[key]), stride) if stride > 1 and ref[key].ndim > 1 else ref[key]) < tol_fw, key
    for key in BW_KEYS + ("dC_initial",):
        if key in got and key in ref:
            assert max_rel_err(subsample(got[key], stride), subsample(np.asarray(ref[key]), stride) if stride > 1 and ref[key].ndim > 1 else ref[key]) < tol_bw, key


@pytest.mark.parametrize("name", [n for n, c in CASES.items() if c["kind"] == "exp_chunkwise"])
def test_exp_f32_vs_reference_golden(name):
    case = CASES[name]
    gold = dict(np.load(os.path.join(GOLD, f"{name}.npz")))
    got = run_cuda_fwbw(make_chunkwise_inputs(case), case["L"])
    compare(got, gold, TOL_F32_FW, TOL_F32_BW, stride=case.get("stride", 1))


@pytest.mark.parametrize("name", ["sig_norm", "sig_nonorm"])
@pytest.mark.parametrize("L", [64, 128])
def test_sig_f32_vs_reference_golden(name, L):
    case = CASES[name]
    gold = dict(np.load(os.path.join(GOLD, f"{name}.npz")))
    got = run_cuda_fwbw(make_chunkwise_inputs(case), L, siging=True, normalize=case["normalize"])
    compare(got, gold, TOL_F32_FW, TOL_F32_BW, keys_fw=("H",))


@pytest.mark.parametrize("normalize", [True, False])
def test_sig_states_vs_reference_golden(normalize):
    """mLSTMsig final states against the values read out of the reference's quadratic implementation."""
    case = CASES["sig_states"]
    gold = dict(np.load(os.path.join(GOLD, "sig_states.npz")))
    got = run_cuda_fwbw(make_chunkwise_inputs(case), case["L"], siging=True, normalize=normalize)
    assert max_rel_err(got["C_last"], gold["C_last"]) < TOL_F32_FW
    if normalize:
        assert max_rel_err(got["n_last"], gold["n_last"]) < TOL_F32_FW


def test_exp_f32_vs_reference_parallel_golden():
    case = CASES["exp_parallel"]
    gold = dict(np.load(os.path.join(GOLD, "exp_parallel.npz")))
    got = run_cuda_fwbw(make_chunkwise_inputs(case), case["L"])
    compare(got, gold, TOL_F32_FW, TOL_F32_BW, keys_fw=("H",))


SHAPES = [
    # B, NH, S, DHQK, DHHV, L
    (1, 2, 64, 32, 64, 16),     # S < 128: one chunk of 64 (reference heuristic)
    (2, 2, 128, 64, 64, 16),
    (1, 3, 256, 48, 96, 32),    # head dims that are not powers of two
    (1, 2, 256, 24, 48, 64),
    (1, 2, 512, 128, 128, 128),
    (1, 1, 512, 64, 128, 256),
    (2, 1, 256, 256, 512, 128),  # decode-model head geometry
]


@pytest.mark.parametrize("shape", SHAPES)
@pytest.mark.parametrize("variant", ["exp", "sig", "sig_nonorm"])
def test_f32_vs_oracle_shapes(shape, variant):
    B, NH, S, DHQK, DHHV, L = shape
    inp = case_inputs(11, B, NH, S, DHQK, DHHV, init=True, dC_last=True)
    siging, normalize = variant != "exp", variant != "sig_nonorm"
    Leff = mk.select_chunk_size(S, L)
    got = run_cuda_fwbw(inp, L, siging=siging, normalize=normalize)
    ref = run_oracle_fwbw(inp, Leff, siging=siging, normalize=normalize)
    keys = FW_KEYS if not siging else (("H", "C_last", "n_last") if normalize else ("H", "C_last"))
    compare(got, ref, TOL_F32_FW, TOL_F32_BW, keys_fw=keys)


@pytest.mark.parametrize("shape", [(2, 2, 256, 64, 128, 64), (1, 2, 512, 128, 128, 128), (1, 2, 256, 256, 256, 128)])
@pytest.mark.parametrize("variant", ["exp", "sig", "sig_nonorm"])
@pytest.mark.parametrize("impl", ["simt", "auto"])
def test_bf16_vs_oracle(shape, variant, impl):
    B, NH, S, DHQK, DHHV, L = shape
    inp = case_inputs(12, B, NH, S, DHQK, DHHV)
    siging, normalize = variant != "exp", variant != "sig_nonorm"
    got = run_cuda_fwbw(inp, L, dtype=torch.bfloat16, siging=siging, normalize=normalize, impl=impl)
    ref = run_oracle_fwbw(inp, L, dtype=torch.bfloat16, siging=siging, normalize=normalize)
    keys = FW_KEYS if not siging else (("H", "C_last", "n_last") if normalize else ("H", "C_last"))
    compare(got, ref, TOL_BF16, TOL_BF16, keys_fw=keys)


@pytest.mark.parametrize("shape", [(1, 1, 256, 512, 512, 128),    # widest qk head the tcgen05 path takes (8 slices)
                                   (1, 1, 256, 128, 1024, 128),   # widest v head (8 output tiles per chunk)
                                   (1, 2, 384, 128, 256, 128),    # odd number of chunks; 128/256 head geometry
                                   (3, 5, 640, 256, 256, 128),    # odd batch x heads, five chunks
                                   (1, 2, 256, 384, 640, 128),    # three and five 128-column tiles per chunk
                                   (1, 2, 384, 64, 64, 128),      # head dims below one tile: zero-padded by TMA
                                   (2, 2, 384, 96, 192, 128),     # 125M-class geometry
                                   (1, 2, 256, 192, 320, 128),    # 1.5 and 2.5 tiles
                                   (1, 1, 256, 72, 136, 128),     # multiples of 8 only
                                   (1, 2, 256, 32, 32, 128),      # a quarter of a tile
                                   (1, 2, 256, 8, 24, 128)])      # the smallest head dims (one 16-byte row)
@pytest.mark.parametrize("variant", ["exp", "sig_nonorm"])
def test_tcgen05_head_geometries(shape, variant):
    """Edge geometries of the tcgen05 path (limits of the head dims it accepts, head dims that are no multiples of its
    128-wide tiles, odd chunk and head counts) against the oracle, with initial states and an incoming state gradient."""
    B, NH, S, DHQK, DHHV, L = shape
    inp = case_inputs(21, B, NH, S, DHQK, DHHV, init=True, dC_last=True)
    siging, normalize = variant != "exp", variant != "sig_nonorm"
    q, v = to_dev(inp["q"], torch.bfloat16), to_dev(inp["v"], torch.bfloat16)
    assert mk.kernel_chunk_size(q, v, L) == 128
    got = run_cuda_fwbw(inp, L, dtype=torch.bfloat16, siging=siging, normalize=normalize, impl="tcgen05")
    ref = run_oracle_fwbw(inp, L, dtype=torch.bfloat16, siging=siging, normalize=normalize)
    keys = FW_KEYS if not siging else ("H", "C_last")
    compare(got, ref, TOL_BF16, TOL_BF16, keys_fw=keys)


@pytest.mark.parametrize("variant", ["exp", "sig"])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_state_passing(variant, dtype):
    """Four segments chained through the returned states equal one pass (reference:
    tests/torch/chunkwise/test_chunkwise_triton_xl_chunk.py:58-72, fixture seed 42 (2,4,256,16,32))."""
    inp = case_inputs(42, 2, 4, 256, 16, 32)
    q, k, v, i, f = (to_dev(inp[n], dtype) for n in "qkvif")
    fn = mk.mlstm_chunkwise__b200_xl_chunk if variant == "exp" else mk.mlstm_siging_chunkwise__b200_xl_chunk
    H_full, last_full = fn(q, k, v, i, f, return_last_states=True, chunk_size=64)
    states = (None,) * (3 if variant == "exp" else 2)
    hs = []
    for s0 in range(0, 256, 64):
        sl = slice(s0, s0 + 64)
        if variant == "exp":
            h, states = fn(q[:, :, sl], k[:, :, sl], v[:, :, sl], i[:, :, sl], f[:, :, sl], states[0], states[1],
                           states[2], return_last_states=True, chunk_size=64)
        else:
            h, states = fn(q[:, :, sl], k[:, :, sl], v[:, :, sl], i[:, :, sl], f[:, :, sl], states[0], states[1],
                           None, return_last_states=True, chunk_size=64)
        hs.append(h)
    tol = 1e-5 if dtype == torch.float32 else 1e-2
    assert max_rel_err(npy(torch.cat(hs, 2)), npy(H_full)) < tol
    # f32 inputs: exact arithmetic on both sides.  bf16 inputs run on the tensor cores, where the four segments gate
    # and round their operands with other chunk boundaries than the single pass (f32 states: 1e-4).
    tol_state = 1e-5 if dtype == torch.float32 else 1e-4
    for a, b in zip(states, last_full):
        assert a.dtype == torch.float32
        assert max_rel_err(npy(a), npy(b)) < tol_state


def test_chunk_size_independence_full_head_dims():
    """H does not depend on the chunk size (size-independent property at the benchmark head geometry
    NH=16-style 256/256, and 256/512)."""
    for DHQK, DHHV in ((256, 256), (256, 512)):
        inp = case_inputs(5, 1, 2, 1024, DHQK, DHHV)
        q, k, v, i, f = (to_dev(inp[n], torch.bfloat16) for n in "qkvif")
        hs = [mk.mlstm_chunkwise__b200_xl_chunk(q, k, v, i, f, chunk_size=L) for L in (64, 128, 256)]
        for h in hs[1:]:
            assert max_rel_err(npy(h), npy(hs[0])) < TOL_BF16


def test_deterministic_and_inputs_untouched():
    inp = case_inputs(3, 1, 2, 512, 128, 128)
    q, k, v, i, f = (to_dev(inp[n], torch.bfloat16) for n in "qkvif")
    q0 = q.clone()
    a = mk.mlstm_chunkwise__b200_xl_chunk(q, k, v, i, f, chunk_size=128)
    b = mk.mlstm_chunkwise__b200_xl_chunk(q, k, v, i, f, chunk_size=128)
    assert torch.equal(a, b)
    assert torch.equal(q, q0)
    assert not torch.isnan(a).any()


def test_return_conventions_and_dtypes():
    inp = case_inputs(4, 1, 2, 128, 32, 64)
    for dt in (torch.float32, torch.bfloat16, torch.float16):
        q, k, v, i, f = (to_dev(inp[n], dt) for n in "qkvif")
        h = mk.mlstm_chunkwise__b200_xl_chunk(q, k, v, i, f)
        assert isinstance(h, torch.Tensor) and h.dtype == dt and h.shape == v.shape
        h, (c, n, m) = mk.mlstm_chunkwise__b200_xl_chunk(q, k, v, i, f, return_last_states=True)
        assert c.shape == (1, 2, 32, 64) and n.shape == (1, 2, 32) and m.shape == (1, 2, 1)
        assert c.dtype == n.dtype == m.dtype == torch.float32 and c.is_contiguous()
        h, st = mk.mlstm_siging_chunkwise__b200_xl_chunk(q, k, v, i, f, return_last_states=True, normalize=False)
        assert len(st) == 2


def test_shape_errors():
    inp = case_inputs(4, 1, 1, 128, 32, 64)
    q, k, v, i, f = (to_dev(inp[n], torch.float32) for n in "qkvif")
    with pytest.raises(ValueError):
        mk.mlstm_chunkwise__b200_xl_chunk(q[:, :, :100], k[:, :, :100], v[:, :, :100], i[:, :, :100], f[:, :, :100])
    with pytest.raises(ValueError):
        mk.mlstm_chunkwise__b200_xl_chunk(q, k, v, i, f, chunk_size=48)
    with pytest.raises(ValueError):
        mk.mlstm_chunkwise__b200_xl_chunk(q, k, v, i, f, autocast_kernel_dtype=torch.float64)
    with pytest.raises(RuntimeError):
        mk.mlstm_chunkwise__b200_xl_chunk(q.cpu(), k.cpu(), v.cpu(), i.cpu(), f.cpu())


def test_autocast_casts_inputs():
    inp = case_inputs(4, 1, 2, 128, 32, 64)
    q, k, v, i, f = (to_dev(inp[n], torch.float32) for n in "qkvif")
    with torch.autocast("cuda", dtype=torch.bfloat16):
        h = mk.mlstm_chunkwise__b200_xl_chunk(q, k, v, i, f, autocast_kernel_dtype=torch.bfloat16)
    assert h.dtype == torch.bfloat16


@pytest.mark.parametrize("variant", ["exp", "sig"])
def test_long_prefill_geometry_chunk256(variant):
    """Head geometry of the long-sequence prefill configuration (NH=8, 256/512, chunk 256), shortened
    sequence.  Chunk sizes above 128 run as chunks of 128 on the tcgen05 path, so the oracle is run at the
    chunk size the kernel used; H is also compared with the oracle at chunk 256 (H does not depend on it)."""
    inp = case_inputs(13, 1, 8, 1024, 256, 512)
    siging = variant != "exp"
    q, k, v = (to_dev(inp[n], torch.bfloat16) for n in "qkv")
    Lk = mk.kernel_chunk_size(q, v, 256)
    assert Lk == 128
    got = run_cuda_fwbw(inp, 256, dtype=torch.bfloat16, siging=siging)
    ref = run_oracle_fwbw(inp, Lk, dtype=torch.bfloat16, siging=siging)
    compare(got, ref, TOL_BF16, TOL_BF16, keys_fw=FW_KEYS if not siging else ("H", "C_last", "n_last"))
    ref256 = run_oracle_fwbw(inp, 256, dtype=torch.bfloat16, siging=siging)
    assert max_rel_err(got["H"], ref256["H"]) < TOL_BF16


def test_forward_backward_capture_in_cuda_graph():
    """The kernels enqueue on the current stream without host synchronisation, so a forward + backward can be captured
    in a CUDA graph and replayed (the reference's callers compile and capture their models)."""
    inp = case_inputs(31, 2, 2, 512, 256, 256)
    q, k, v = (to_dev(inp[n], torch.bfloat16) for n in "qkv")
    i, f = (to_dev(inp[n], torch.float32) for n in "if")
    dh = to_dev(inp["dH"], torch.float32)

    def step():
        # leaves and the gradient seed are created inside the step, on the stream it runs on: autograd would otherwise
        # synchronise with the stream that created them, which a capture does not allow
        leaves = [t.detach().requires_grad_(True) for t in (q, k, v, i, f)]
        h = mk.mlstm_chunkwise__b200_xl_chunk(*leaves, chunk_size=128)
        grads = torch.autograd.grad((h.float() * dh).sum(), leaves)
        return (h.detach(),) + grads

    eager = [t.clone() for t in step()]
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):       # warm-up on a side stream, as graph capture requires
        step()
    torch.cuda.current_stream().wait_stream(side)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        outs = step()
    for _ in range(2):
        graph.replay()
    torch.cuda.synchronize()
    for a, b in zip(eager, outs):
        assert torch.equal(a, b)


@pytest.mark.parametrize("dtype,dims,L,S", [(torch.bfloat16, (256, 256), 128, 1024), (torch.float32, (32, 64), 64, 512)])
@pytest.mark.parametrize("gates", [(8.0, 0.0), (4.0, -6.0), (1.0, 12.0)])
@pytest.mark.parametrize("variant", ["exp", "sig"])
def test_extreme_gate_values(dtype, dims, L, S, gates, variant):
    """Gate pre-activations far outside the benchmark's distribution: input gates 8 N(0,1) (single tokens dominate a
    whole chunk), forget gates around -6 (the state is wiped at nearly every step) and around +12 (nothing decays).
    Nothing may overflow or lose the stabilisation.  Tolerance: f32 1e-3; bf16 3e-2 - with a handful of dominant terms
    per output the bf16 roundings of the gated tile no longer average out (the same inputs in fp16 give 1e-3)."""
    scale, offset = gates
    inp = case_inputs(77, 1, 2, S, dims[0], dims[1])
    rng = np.random.default_rng(5)
    inp["i"] = (scale * rng.standard_normal(inp["i"].shape)).astype(np.float32)
    inp["f"] = (offset + scale * rng.standard_normal(inp["f"].shape)).astype(np.float32)
    siging = variant == "sig"
    got = run_cuda_fwbw(inp, L, dtype=dtype, siging=siging)
    ref = run_oracle_fwbw(inp, L, dtype=dtype, siging=siging)
    tol = 1e-3 if dtype == torch.float32 else 3e-2
    for key in ("H", "C_last", "dQ", "dK", "dV", "dI", "dF"):
        assert np.isfinite(got[key]).all(), key
        assert max_rel_err(got[key], ref[key]) < tol, key


@pytest.mark.parametrize("recompute", [True, False])
@pytest.mark.parametrize("odd", [False, True])
def test_two_stream_unit_split_is_bit_identical_and_capturable(odd, recompute):
    """With more recurrence CTAs than SMs and a poorly filled last wave, the library runs the two halves of the
    (batch, head) units on two streams.  Same kernels on the same data: every output must be bit-identical to the
    single-stream run, with an odd number of units too and with either way of getting the per-chunk states in the
    backward (kept, or recomputed inside the launch chains), and the forked launches must survive a graph capture."""
    from mlstm_kernels_b200 import _lib
    lib = _lib.load()
    B, NH = (3, 67) if odd else (2, 100)          # 201 / 200 state tiles of 128 x 128 on 148 SMs: two waves, 68 % full
    g = torch.Generator(device="cuda").manual_seed(11)
    rnd = lambda *s: torch.randn(*s, device="cuda", generator=g)  # noqa: E731
    q, k, v = (rnd(B, NH, 300, 128).bfloat16() for _ in range(3))
    i, f = rnd(B, NH, 300).bfloat16(), (3 + rnd(B, NH, 300)).bfloat16()
    dh = rnd(B, NH, 300, 128).bfloat16()

    def step():
        leaves = [t.detach().requires_grad_(True) for t in (q, k, v, i, f)]
        h, last = mk.mlstm_chunkwise__b200_xl_chunk(*leaves, chunk_size=128, return_last_states=True,
                                                    recompute_states_in_bw=recompute)
        grads = torch.autograd.grad(h, leaves, dh)
        return (h.detach(),) + tuple(last) + grads

    prev = lib.mlstm_b200_set_unit_split(0)
    try:
        single = [t.clone() for t in step()]
        lib.mlstm_b200_set_unit_split(1)
        split = [t.clone() for t in step()]
        for a, b in zip(single, split):
            assert torch.equal(a, b)
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            step()
        torch.cuda.current_stream().wait_stream(side)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            outs = step()
        for _ in range(2):
            graph.replay()
        torch.cuda.synchronize()
        for a, b in zip(single, outs):
            assert torch.equal(a, b)
    finally:
        lib.mlstm_b200_set_unit_split(prev)


def test_benchmark_size_properties():
    """At the benchmark size (B=8, S=8192, NH=16, 256/256, bf16: too large for the oracle) the kernels are checked
    through properties that do not depend on the size: reruns are bit-identical (forward and all five gradients),
    a (batch, head) slice computed alone gives bit-identical results (units are independent), the sequence processed
    as two halves with state passing reproduces H and the final state, and a sub-block is checked against the oracle."""
    B, NH, S, D, L = 8, 16, 8192, 256, 128
    g = torch.Generator(device="cuda").manual_seed(5)
    rnd = lambda *s: torch.randn(*s, device="cuda", generator=g)  # noqa: E731
    q, k, v = (rnd(B, NH, S, D).bfloat16() for _ in range(3))
    i, f = rnd(B, NH, S).bfloat16(), (3 + rnd(B, NH, S)).bfloat16()
    dh = rnd(B, NH, S, D).bfloat16()

    def fwbw(qq, kk, vv, ii, ff, dd):
        leaves = [t.detach().clone().requires_grad_(True) for t in (qq, kk, vv, ii, ff)]
        h, last = mk.mlstm_chunkwise__b200_xl_chunk(*leaves, return_last_states=True, chunk_size=L)
        h.backward(dd)
        return [h.detach()] + [t.grad for t in leaves], last

    a, last_a = fwbw(q, k, v, i, f, dh)
    b, _ = fwbw(q, k, v, i, f, dh)
    for x, y in zip(a, b):
        assert torch.equal(x, y)
        assert torch.isfinite(x.float()).all()
    # one (batch, head) unit on its own
    sl = (slice(5, 6), slice(11, 12))
    c, _ = fwbw(*(t[sl].contiguous() for t in (q, k, v, i, f, dh)))
    for x, y in zip(a, c):
        assert torch.equal(x[sl], y)
    # two halves with state passing
    hlf = S // 2
    first = [t[:, :, :hlf].contiguous() for t in (q, k, v, i, f)]
    second = [t[:, :, hlf:].contiguous() for t in (q, k, v, i, f)]
    with torch.no_grad():
        h1, st = mk.mlstm_chunkwise__b200_xl_chunk(*first, return_last_states=True, chunk_size=L)
        h2, st2 = mk.mlstm_chunkwise__b200_xl_chunk(*second, c_initial=st[0], n_initial=st[1], m_initial=st[2],
                                                    return_last_states=True, chunk_size=L)
    assert torch.equal(torch.cat([h1, h2], 2), a[0])
    for x, y in zip(st2, last_a):
        assert max_rel_err(npy(x), npy(y)) < 1e-5
    # the single unit against the oracle (forward and gradients)
    unit = {n: npy(t[sl]) for n, t in zip(("q", "k", "v", "i", "f", "dH"), (q, k, v, i, f, dh))}
    ref_fw, ref_bw = O.chunkwise_fwbw(unit["q"], unit["k"], unit["v"], unit["i"], unit["f"], unit["dH"], chunk_size=L)
    assert max_rel_err(npy(c[0]), ref_fw["H"]) < TOL_BF16
    for j, key in enumerate(("dQ", "dK", "dV", "dI", "dF"), start=1):
        assert max_rel_err(npy(c[j]), ref_bw[key]) < TOL_BF16, key


@pytest.mark.parametrize("variant", ["exp", "sig"])
@pytest.mark.parametrize("impl,dtype,shape", [("auto", torch.bfloat16, (2, 2, 512, 256, 256, 128)),
                                              ("simt", torch.float32, (1, 2, 256, 64, 128, 64))])
def test_recompute_states_in_bw(variant, impl, dtype, shape):
    """recompute_states_in_bw=True (the reference's default: the per-chunk states are not kept, the backward runs the
    recurrence again) and False (states kept) give bit-identical outputs and gradients, both match the oracle, and the
    recompute setting holds less memory between forward and backward (by the size of the state buffer)."""
    B, NH, S, DHQK, DHHV, L = shape
    inp = case_inputs(41, B, NH, S, DHQK, DHHV, init=True, dC_last=True)
    siging = variant != "exp"
    fn = mk.mlstm_siging_chunkwise__b200_xl_chunk if siging else mk.mlstm_chunkwise__b200_xl_chunk
    def run(rc):
        leaves = [to_dev(inp[n], dtype, True) for n in "qkvif"]
        c0 = to_dev(inp["c0"], torch.float32, True)
        n0, m0 = to_dev(inp["n0"], torch.float32), to_dev(inp["m0"], torch.float32)
        dh, dcl = to_dev(inp["dH"], torch.float32), to_dev(inp["dC_last"], torch.float32)
        torch.cuda.synchronize()
        base = torch.cuda.memory_allocated()
        h, last = fn(*leaves, c0, n0, None if siging else m0, True, chunk_size=L, impl=impl,
                     recompute_states_in_bw=rc)
        torch.cuda.synchronize()
        held_bytes = torch.cuda.memory_allocated() - base     # outputs + what autograd keeps for the backward
        loss = (h.float() * dh).sum() + (last[0] * dcl).sum()
        loss.backward()
        return [npy(h)] + [npy(t.grad) for t in leaves] + [npy(c0.grad)], held_bytes

    res, held = {}, {}
    for rc in (True, False):
        res[rc], held[rc] = run(rc)
    for a, b in zip(res[True], res[False]):
        assert np.array_equal(a, b)
    state_bytes = B * NH * (S // L + 1) * DHQK * DHHV * (2 if impl == "auto" else 4)
    assert held[False] - held[True] >= 0.9 * state_bytes
    ref = run_oracle_fwbw(inp, L, dtype=dtype, siging=siging)
    tol_fw, tol_bw = (TOL_BF16, TOL_BF16) if dtype == torch.bfloat16 else (TOL_F32_FW, TOL_F32_BW)
    got = dict(zip(("H", "dQ", "dK", "dV", "dI", "dF", "dC_initial"), res[True]))
    compare(got, ref, tol_fw, tol_bw, keys_fw=("H",))


@pytest.mark.parametrize("shape", [(2, 3, 200, 72, 136), (1, 2, 384, 256, 256), (2, 2, 96, 16, 32)])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_every_output_element_is_written(shape, dtype):
    """Outputs are allocated uninitialised.  The allocator's free blocks are filled with NaN first, so an element a
    kernel forgot to write (a masked tail, a tile edge) would surface as NaN in H, the states or a gradient."""
    B, NH, S, DHQK, DHHV = shape
    if dtype == torch.float32 and S % 64 != 0:
        S = 192   # the portable kernels need whole chunks
    inp = case_inputs(5, B, NH, S, DHQK, DHHV, init=True, dC_last=True)
    torch.cuda.synchronize()
    poison = [torch.full((64 << 20,), float("nan"), device="cuda") for _ in range(4)]   # 1 GiB of NaN
    small = [torch.full((n,), float("nan"), device="cuda") for n in (1 << 10, 1 << 14, 1 << 18, 1 << 20) for _ in range(8)]
    torch.cuda.synchronize()
    del poison, small
    got = run_cuda_fwbw(inp, 64, dtype=dtype)
    for key, val in got.items():
        assert np.isfinite(val).all(), key


def test_nvtx_ranges_do_not_change_results():
    """NVTX ranges around the phases are host-side markers: switched on (no profiler attached) a forward + backward
    gives the same bits, and the setter returns the previous setting."""
    from mlstm_kernels_b200 import _lib
    lib = _lib.load()
    inp = case_inputs(3, 1, 2, 256, 128, 128)
    off = run_cuda_fwbw(inp, 128, dtype=torch.bfloat16)
    prev = lib.mlstm_b200_nvtx_enable(1)
    try:
        on = run_cuda_fwbw(inp, 128, dtype=torch.bfloat16)
        assert lib.mlstm_b200_nvtx_enable(1) == 1
    finally:
        lib.mlstm_b200_nvtx_enable(prev)
    for key in off:
        assert np.array_equal(off[key], on[key]), key


def test_bounded_wait_expiry_is_reported():
    """A wait that runs out records its code in the device status word and the context stays usable.  The self-test
    kernel waits a few thousand polls on a barrier that nothing signals (no copy in flight, no tensor memory held),
    gives up and returns; afterwards the word is cleared and a normal forward runs and leaves it at 0."""
    from mlstm_kernels_b200 import _lib
    lib = _lib.load()
    assert _lib.device_status() == 0
    assert lib.mlstm_b200_selftest_wait_expiry(2000, 901, None) == 0
    assert _lib.device_status(reset=False) == 901
    assert lib.mlstm_b200_selftest_wait_expiry(2000, 902, None) == 0
    assert _lib.device_status(reset=True) == 901        # the FIRST code is kept until the word is cleared
    assert _lib.device_status() == 0
    assert lib.mlstm_b200_selftest_wait_expiry(0, 901, None) == -7          # limits outside 1 .. 1e6 are refused
    assert lib.mlstm_b200_selftest_wait_expiry(5_000_000, 901, None) == -7
    # an expired wait does not poison later launches: the status word is never read by a kernel
    assert lib.mlstm_b200_selftest_wait_expiry(2000, 903, None) == 0
    inp = case_inputs(43, 1, 2, 256, 256, 256)
    got = run_cuda_fwbw(inp, 128, dtype=torch.bfloat16, impl="tcgen05")
    ref = run_oracle_fwbw(inp, 128, dtype=torch.bfloat16)
    compare(got, ref, TOL_BF16, TOL_BF16)
    assert _lib.device_status(reset=True) == 903


def _random_geometries(count, seed):
    rng = np.random.default_rng(seed)
    out = []
    for _ in range(count):
        B, NH = int(rng.integers(1, 4)), int(rng.integers(1, 4))
        S = int(rng.integers(1, 420))
        DHQK, DHHV = 8 * int(rng.integers(1, 41)), 8 * int(rng.integers(1, 49))   # 8 .. 320, 8 .. 384
        out.append((B, NH, S, DHQK, DHHV, ["exp", "sig", "sig_nonorm"][int(rng.integers(0, 3))]))
    return out


@pytest.mark.parametrize("geom", _random_geometries(24, 2024))
def test_tcgen05_random_geometries(geom):
    """Randomly drawn (seeded) batch, heads, sequence length (any) and head dims (any multiples of 8): every
    combination of ragged tokens and head dims off the 128-wide tiles, with initial states and an incoming state
    gradient, against the oracle (run with a chunk size that divides S)."""
    B, NH, S, DHQK, DHHV, variant = geom
    inp = case_inputs(1000 + S, B, NH, S, DHQK, DHHV, init=True, dC_last=True)
    siging, normalize = variant != "exp", variant != "sig_nonorm"
    got = run_cuda_fwbw(inp, 128, dtype=torch.bfloat16, siging=siging, normalize=normalize, impl="tcgen05")
    ref = run_oracle_fwbw(inp, _largest_divisor_up_to(S, 128), dtype=torch.bfloat16, siging=siging, normalize=normalize)
    compare(got, ref, TOL_BF16, TOL_BF16, keys_fw=("H",))
    if siging:
        assert max_rel_err(got["C_last"], ref["C_last"]) < TOL_BF16
    else:
        sg, sr = np.exp(got["m_last"]), np.exp(ref["m_last"])
        assert max_rel_err(got["C_last"] * sg[..., None], ref["C_last"] * sr[..., None]) < TOL_BF16
        assert max_rel_err(got["n_last"] * sg, ref["n_last"] * sr) < TOL_BF16


def _largest_divisor_up_to(n, cap):
    return max(d for d in range(1, cap + 1) if n % d == 0)


@pytest.mark.parametrize("shape", [(2, 2, 300, 128, 128), (1, 2, 64, 256, 256), (1, 2, 448, 128, 256),
                                   (1, 1, 129, 256, 256), (1, 2, 1000, 128, 128), (2, 1, 17, 128, 128),
                                   (2, 2, 300, 96, 192), (1, 2, 77, 64, 200)])   # ragged in tokens AND head dims
@pytest.mark.parametrize("variant", ["exp", "sig", "sig_nonorm"])
def test_tcgen05_any_sequence_length(shape, variant):
    """On the tcgen05 path the sequence length need not be a multiple of the chunk size (nor of 16): the last chunk
    is ragged, its missing tokens are read as zeros and switched off in the gates, and no row past S is written.
    Checked against the oracle run with a chunk size that divides S (H and the gradients do not depend on the chunk
    size; the (C, n, m) triple is compared through C exp(m), n exp(m)), with initial states and an incoming state
    gradient."""
    B, NH, S, DHQK, DHHV = shape
    inp = case_inputs(71, B, NH, S, DHQK, DHHV, init=True, dC_last=(variant != "exp"))
    siging, normalize = variant != "exp", variant != "sig_nonorm"
    q, v = to_dev(inp["q"], torch.bfloat16), to_dev(inp["v"], torch.bfloat16)
    assert mk.resolve_chunk_size(q, v, 64) == 128
    got = run_cuda_fwbw(inp, 64, dtype=torch.bfloat16, siging=siging, normalize=normalize)
    assert got["H"].shape == (B, NH, S, DHHV) and got["dF"].shape == (B, NH, S)
    ref = run_oracle_fwbw(inp, _largest_divisor_up_to(S, 128), dtype=torch.bfloat16, siging=siging, normalize=normalize)
    compare(got, ref, TOL_BF16, TOL_BF16, keys_fw=("H",))
    if siging:
        assert max_rel_err(got["C_last"], ref["C_last"]) < TOL_BF16
        if normalize:
            assert max_rel_err(got["n_last"], ref["n_last"]) < TOL_BF16
    else:
        sg, sr = np.exp(got["m_last"]), np.exp(ref["m_last"])
        assert max_rel_err(got["C_last"] * sg[..., None], ref["C_last"] * sr[..., None]) < TOL_BF16
        assert max_rel_err(got["n_last"] * sg, ref["n_last"] * sr) < TOL_BF16


def test_ragged_tail_writes_nothing_past_the_sequence():
    """The (batch, head) blocks of an output are contiguous, so a row written past the last token of one head would
    land in the first rows of the next head.  Each head computed alone must therefore reproduce its block of the
    joint run bit for bit."""
    B, NH, S, D = 1, 3, 200, 128
    inp = case_inputs(72, B, NH, S, D, D)
    full = run_cuda_fwbw(inp, 128, dtype=torch.bfloat16)
    for h in range(NH):
        one = {n: x[:, h:h + 1] for n, x in inp.items()}
        alone = run_cuda_fwbw(one, 128, dtype=torch.bfloat16)
        for key in ("H", "dQ", "dK", "dV", "dI", "dF"):
            assert np.array_equal(full[key][:, h:h + 1], alone[key]), (h, key)


@pytest.mark.parametrize("shape", [(2, 2, 512, 256, 256), (1, 2, 300, 128, 256), (1, 1, 1024, 256, 512)])
@pytest.mark.parametrize("variant", ["exp", "sig", "sig_nonorm"])
def test_tcgen05_fp16(shape, variant):
    """IEEE half inputs take the tensor-core path as well (f16 operands, f16 per-chunk states, f32 accumulation):
    against the oracle on the f16-rounded inputs, with initial states, an incoming state gradient and a ragged length.
    f16 carries three more mantissa bits than bf16, so the bound is tighter: 2e-3 (measured 2-6e-4)."""
    B, NH, S, DHQK, DHHV = shape
    inp = case_inputs(81, B, NH, S, DHQK, DHHV, init=True, dC_last=True)
    siging, normalize = variant != "exp", variant != "sig_nonorm"
    q, v = to_dev(inp["q"], torch.float16), to_dev(inp["v"], torch.float16)
    assert mk.tcgen05_applies(q, v)
    got = run_cuda_fwbw(inp, 128, dtype=torch.float16, siging=siging, normalize=normalize, impl="tcgen05")
    ref = run_oracle_fwbw(inp, _largest_divisor_up_to(S, 128), dtype=torch.float16, siging=siging, normalize=normalize)
    worst = {k_: max_rel_err(got[k_], ref[k_]) for k_ in ("H", "dQ", "dK", "dV", "dI", "dF", "dC_initial")}
    print("\nfp16", shape, variant, {k_: f"{e:.2e}" for k_, e in worst.items()})
    compare(got, ref, 2e-3, 2e-3, keys_fw=("H",))
    if siging:
        assert max_rel_err(got["C_last"], ref["C_last"]) < 2e-3
    else:
        sg, sr = np.exp(got["m_last"]), np.exp(ref["m_last"])
        assert max_rel_err(got["C_last"] * sg[..., None], ref["C_last"] * sr[..., None]) < 2e-3
