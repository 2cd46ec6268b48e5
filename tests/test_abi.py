"""CPU-side checks of the C-ABI library: it loads, exports every symbol the header declares, and
rejects bad arguments before touching the GPU."""

import ctypes
import os
import re

import pytest

from mlstm_kernels_b200 import _lib, select_chunk_size

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "mlstm_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(mlstm_b200_\w+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    lib = _lib.load()
    names = declared_symbols()
    assert len(names) >= 10
    for name in names:
        assert hasattr(lib, name), name
        assert name in _lib.SIGNATURES, f"{name} has no ctypes signature"
    assert lib.mlstm_b200_version() >= 100


def test_error_strings_and_argument_validation():
    lib = _lib.load()
    assert lib.mlstm_b200_error_string(0) == b"ok"
    assert b"workspace" in lib.mlstm_b200_error_string(-5)
    # sizes are validated before any CUDA call: S not divisible by L, L not a power of two
    assert lib.mlstm_b200_chunkwise_workspace_bytes(1, 1, 100, 64, 64, 64, 0, 0, 0, 0) == 0
    assert lib.mlstm_b200_chunkwise_workspace_bytes(1, 1, 96, 64, 64, 48, 0, 0, 0, 0) == 0
    assert lib.mlstm_b200_chunkwise_workspace_bytes(2, 4, 512, 128, 256, 64, 0, 0, 0, 0) > 0
    # sizes whose grids or 32-bit row coordinates would overflow are refused, not launched
    assert lib.mlstm_b200_chunkwise_workspace_bytes(65536, 64, 1 << 20, 128, 128, 128, 1, 0, 0, 0) == 0
    # the removed implementation code is rejected
    assert lib.mlstm_b200_chunkwise_state_dtype(256, 256, 256, 128, 1, 3) == 0
    null = ctypes.c_void_p(None)
    rc = lib.mlstm_b200_step(*([null] * 12), 1, 1, 64, 64, 0, 0, 0, 1e-6, null)
    assert rc == -3  # MLSTM_ERR_NULL
    rc = lib.mlstm_b200_step(*([null] * 12), 1, 1, 64, 66, 0, 0, 0, 1e-6, null)
    assert rc == -1  # MLSTM_ERR_SHAPE


def test_select_chunk_size_follows_reference_heuristic():
    assert select_chunk_size(64, 128) == 64      # short sequences run as one chunk
    assert select_chunk_size(512, 128) == 128
    assert select_chunk_size(512, 32) == 32
    with pytest.raises(ValueError):
        select_chunk_size(100, 64)
    with pytest.raises(ValueError):
        select_chunk_size(96, 64)
    with pytest.raises(ValueError):
        select_chunk_size(384, 256)


def test_cpu_tensors_are_rejected():
    import torch

    import mlstm_kernels_b200 as mk
    q = torch.zeros(1, 1, 64, 32)
    with pytest.raises(RuntimeError):
        mk.mlstm_chunkwise__b200_xl_chunk(q, q, q, q[..., 0], q[..., 0])
    with pytest.raises(RuntimeError):
        mk.mlstm_recurrent_step__b200(q[:, :, 0], q[:, :, 0], q[:, :, 0], q[:, :, 0, :1], q[:, :, 0, :1],
                                      torch.zeros(1, 1, 32, 32), torch.zeros(1, 1, 32), torch.zeros(1, 1, 1))
