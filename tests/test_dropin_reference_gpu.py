"""Drop-in check against the reference package itself, when it is importable on the test machine
(e.g. installed with `pip install --no-deps --target baseline/_ref <reference checkout>`); skipped otherwise.
The B200 kernels are registered in the reference's registries and driven through its own, unmodified
mLSTMBackend (train and inference modes, arbitrary sequence length, padding) and compared with the reference's
native PyTorch kernels run on the same GPU."""

import os
import sys

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
_ref = os.path.join(ROOT, "baseline", "_ref")
if os.path.isdir(_ref) and _ref not in sys.path:
    sys.path.insert(0, _ref)
pytest.importorskip("mlstm_kernels")

import mlstm_kernels_b200 as mk  # noqa: E402
from inputs import max_rel_err  # noqa: E402
from util_gpu import case_inputs, npy, to_dev  # noqa: E402

pytestmark = pytest.mark.gpu


def _backend(chunkwise, mode, **kw):
    from mlstm_kernels.torch.backend_module import mLSTMBackend, mLSTMBackendConfig
    return mLSTMBackend(mLSTMBackendConfig(chunkwise_kernel=chunkwise, mode=mode, **kw))


def test_registration_and_names():
    assert mk.register_with_mlstm_kernels()
    from mlstm_kernels.torch import get_available_mlstm_kernels, get_available_mlstm_step_kernels
    assert "chunkwise--b200_xl_chunk" in get_available_mlstm_kernels()
    assert "b200" in get_available_mlstm_step_kernels()


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 1e-4), (torch.bfloat16, 2e-2)])
def test_backend_train_mode_matches_native(dtype, tol):
    mk.register_with_mlstm_kernels()
    inp = case_inputs(51, 2, 2, 256, 128, 128)
    q, k, v, i, f = (to_dev(inp[n], dtype) for n in "qkvif")
    kw = dict(chunk_size=128, return_last_states=True, autocast_kernel_dtype="float32")
    h_b, st_b = _backend("chunkwise--b200_xl_chunk", "train", **kw)(q, k, v, i, f)
    h_n, st_n = _backend("chunkwise--native_custbw", "train", **kw)(q.float(), k.float(), v.float(), i.float(), f.float())
    assert max_rel_err(npy(h_b), npy(h_n)) < tol
    assert max_rel_err(npy(st_b[0]), npy(st_n[0])) < tol


@pytest.mark.parametrize("S", [65, 93, 200, 500])
def test_backend_inference_arbitrary_length(S):
    """The reference's arbitrary-sequence-length wrapper (mlstm_kernels/torch/kernel_wrappers.py:12-203) drives the
    B200 chunkwise kernel with chunk sizes 64..16, then the sequence kernel for the tail."""
    mk.register_with_mlstm_kernels()
    inp = case_inputs(52, 1, 2, 512, 64, 128)
    q, k, v, i, f = (to_dev(inp[n][:, :, :S], torch.float32) for n in "qkvif")
    kw = dict(chunk_size=64, return_last_states=True, inference_state_dtype="float32")
    h_b, st_b = _backend("chunkwise--b200_xl_chunk", "inference", sequence_kernel="native_sequence__b200",
                         step_kernel="b200", **kw)(q, k, v, i, f)
    h_n, st_n = _backend("chunkwise--native_custbw", "inference", sequence_kernel="native_sequence__native",
                         step_kernel="native", **kw)(q, k, v, i, f)
    assert h_b.shape == (1, 2, S, 128)
    assert max_rel_err(npy(h_b), npy(h_n)) < 1e-4
    # (C, n, m) agree up to the common stabiliser scale exp(m)
    sb = st_b[0] * torch.exp(st_b[2])[..., None]
    sn = st_n[0] * torch.exp(st_n[2])[..., None]
    assert max_rel_err(npy(sb), npy(sn)) < 1e-4


@pytest.mark.parametrize("S", [93, 500, 777])
def test_backend_inference_arbitrary_length_tensor_cores(S):
    """Same wrapper, bf16 and head dims that the tcgen05 kernels take: every chunk size of the wrapper's ladder
    (64, 32, 16) runs on the tensor cores as ragged 128-token chunks.  Compared with the reference's native kernels
    in f32 on the same (bf16-rounded) inputs."""
    mk.register_with_mlstm_kernels()
    inp = case_inputs(55, 1, 2, 1024, 128, 256)
    q, k, v, i, f = (to_dev(inp[n][:, :, :S], torch.bfloat16) for n in "qkvif")
    kw = dict(chunk_size=64, return_last_states=True, inference_state_dtype="float32")
    h_b, st_b = _backend("chunkwise--b200_xl_chunk", "inference", sequence_kernel="native_sequence__b200",
                         step_kernel="b200", **kw)(q, k, v, i, f)
    h_n, st_n = _backend("chunkwise--native_custbw", "inference", sequence_kernel="native_sequence__native",
                         step_kernel="native", **kw)(q.float(), k.float(), v.float(), i.float(), f.float())
    assert h_b.shape == (1, 2, S, 256) and h_b.dtype == torch.bfloat16
    assert max_rel_err(npy(h_b), npy(h_n)) < 2e-2
    sb = st_b[0] * torch.exp(st_b[2])[..., None]
    sn = st_n[0] * torch.exp(st_n[2])[..., None]
    assert max_rel_err(npy(sb), npy(sn)) < 2e-2


def test_train_mode_any_length_without_padding():
    """mode="train" with a sequence length that is no multiple of the chunk size: the B200 kernel masks the ragged
    tail itself, so the host-side zero-padding copies of mode="train_with_padding" are not needed; both give the
    reference's padded result."""
    mk.register_with_mlstm_kernels()
    inp = case_inputs(56, 2, 2, 512, 128, 128)
    q, k, v, i, f = (to_dev(inp[n][:, :, :300], torch.bfloat16) for n in "qkvif")
    kw = dict(chunk_size=128, return_last_states=False)
    h_direct = _backend("chunkwise--b200_xl_chunk", "train", **kw)(q, k, v, i, f)
    h_padded = _backend("chunkwise--b200_xl_chunk", "train_with_padding", **kw)(q, k, v, i, f)
    h_n = _backend("chunkwise--native_custbw", "train_with_padding", **kw)(q.float(), k.float(), v.float(), i.float(), f.float())
    assert h_direct.shape == (2, 2, 300, 128)
    assert max_rel_err(npy(h_direct), npy(h_n)) < 2e-2
    assert max_rel_err(npy(h_padded), npy(h_n)) < 2e-2
    assert max_rel_err(npy(h_direct), npy(h_padded)) < 1e-2


def test_backend_train_with_padding():
    mk.register_with_mlstm_kernels()
    inp = case_inputs(53, 1, 2, 512, 64, 128)
    q, k, v, i, f = (to_dev(inp[n][:, :, :300], torch.float32) for n in "qkvif")
    kw = dict(chunk_size=128, return_last_states=False)
    h_b = _backend("chunkwise--b200_xl_chunk", "train_with_padding", **kw)(q, k, v, i, f)
    h_n = _backend("chunkwise--native_custbw", "train_with_padding", **kw)(q, k, v, i, f)
    assert h_b.shape == (1, 2, 300, 128)
    assert max_rel_err(npy(h_b), npy(h_n)) < 1e-4


def test_single_step_through_backend():
    mk.register_with_mlstm_kernels()
    inp = case_inputs(54, 2, 2, 16, 64, 128)
    q, k, v, i, f = (to_dev(inp[n][:, :, :1], torch.float32) for n in "qkvif")
    c0 = torch.randn(2, 2, 64, 128, device="cuda") * 0.1
    n0 = torch.randn(2, 2, 64, device="cuda").abs()
    m0 = torch.randn(2, 2, 1, device="cuda")
    kw = dict(chunk_size=64, return_last_states=True, inference_state_dtype="float32")
    h_b, st_b = _backend("chunkwise--b200_xl_chunk", "inference", step_kernel="b200", **kw)(q, k, v, i, f, c0, n0, m0)
    h_n, st_n = _backend("chunkwise--native_custbw", "inference", step_kernel="native", **kw)(q, k, v, i, f, c0, n0, m0)
    assert max_rel_err(npy(h_b), npy(h_n)) < 1e-5
    assert max_rel_err(npy(st_b[0]), npy(st_n[0])) < 1e-5


@pytest.mark.parametrize("mode", ["train", "inference"])
def test_backend_module_under_torch_compile(mode):
    """The reference's own backend module, compiled, with the B200 kernels inside (no graph break allowed): same bits
    as the eager module.  bf16, ragged length in inference mode (one chunkwise call on the tensor-core path)."""
    mk.register_with_mlstm_kernels()
    S = 256 if mode == "train" else 300
    inp = case_inputs(53, 2, 2, 512, 128, 128)
    q, k, v, i, f = (to_dev(inp[n][:, :, :S], torch.bfloat16) for n in "qkvif")
    kw = dict(chunk_size=128, return_last_states=True, autocast_kernel_dtype="bfloat16")
    if mode == "inference":
        kw.update(sequence_kernel="native_sequence__b200", step_kernel="b200", inference_state_dtype="float32")
    backend = _backend("chunkwise--b200_xl_chunk", mode, **kw)
    h_e, st_e = backend(q, k, v, i, f)
    h_c, st_c = torch.compile(backend, fullgraph=True)(q, k, v, i, f)
    assert torch.equal(h_e, h_c)
    for a, b in zip(st_e, st_c):
        assert torch.equal(a, b)
