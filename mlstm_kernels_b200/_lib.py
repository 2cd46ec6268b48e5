"""ctypes binding of libmlstm_b200.so (the C ABI declared in include/mlstm_b200.h).

There is no fallback: if the shared library is missing or a call fails, an exception is raised.
"""

from __future__ import annotations

import ctypes as C
import os

import torch

_PKG = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_PKG, "libmlstm_b200.so")

F32, BF16, F16 = 0, 1, 2
EXP, SIG, SIG_NONORM = 0, 1, 2
IMPL = {"auto": 0, "simt": 1, "tcgen05": 2}

_DTYPE_CODE = {torch.float32: F32, torch.bfloat16: BF16, torch.float16: F16}
_CODE_DTYPE = {v: k for k, v in _DTYPE_CODE.items()}

_vp, _fp, _i, _f, _sz = C.c_void_p, C.c_void_p, C.c_int, C.c_float, C.c_size_t

# name -> (restype, argtypes); must list every symbol declared in include/mlstm_b200.h
SIGNATURES = {
    "mlstm_b200_version": (_i, []),
    "mlstm_b200_error_string": (C.c_char_p, [_i]),
    "mlstm_b200_last_cuda_error": (C.c_char_p, []),
    "mlstm_b200_launch_count": (C.c_longlong, []),
    "mlstm_b200_device_status": (_i, [_i]),
    "mlstm_b200_selftest_wait_expiry": (_i, [C.c_uint, _i, _vp]),
    "mlstm_b200_profile_enable": (_i, [_i]),
    "mlstm_b200_profile_phases": (_i, []),
    "mlstm_b200_profile_phase_name": (C.c_char_p, [_i]),
    "mlstm_b200_profile_read": (_i, [C.POINTER(C.c_float), C.POINTER(C.c_int)]),
    "mlstm_b200_chunkwise_has_tcgen05": (_i, [_i] * 5),
    "mlstm_b200_chunkwise_state_dtype": (_i, [_i] * 6),
    "mlstm_b200_chunkwise_workspace_bytes": (_sz, [_i] * 10),
    "mlstm_b200_chunkwise_fw": (_i, [_vp] * 5 + [_fp] * 3 + [_vp, _fp, _fp] + [_vp, _fp, _fp] + [_fp] * 3
                                + [_vp, _sz] + [_i] * 6 + [_i, _i, _i, _i, _f, _vp]),
    "mlstm_b200_static_scratch_bytes": (_sz, []),
    "mlstm_b200_static_warmup": (_i, []),
    "mlstm_b200_chunkwise_fw_static": (_i, [_vp] * 5 + [_fp] * 3 + [_vp, _fp, _fp] + [_vp, _fp, _fp] + [_fp] * 3
                                       + [_i] * 6 + [_i, _i, _i, _i, _f, _vp]),
    "mlstm_b200_chunkwise_bw": (_i, [_vp] * 5 + [_fp, _vp, _fp, _vp, _fp] + [_vp] * 3 + [_fp] * 3
                                + [_vp, _sz] + [_i] * 6 + [_i, _i, _i, _i, _f, _vp]),
    "mlstm_b200_chunkwise_bw_cached": (_i, [_vp] * 5 + [_fp, _vp, _fp, _fp, _vp, _sz, _vp, _fp] + [_vp] * 3 + [_fp] * 3
                                       + [_vp, _sz] + [_i] * 6 + [_i, _i, _i, _i, _f, _vp]),
    "mlstm_b200_chunkwise_bw_recompute": (_i, [_vp] * 5 + [_fp, _fp, _vp, _fp, _fp, _vp, _sz, _vp, _fp] + [_vp] * 3
                                          + [_fp] * 3 + [_vp, _sz] + [_i] * 6 + [_i, _i, _i, _i, _f, _vp]),
    "mlstm_b200_chunkwise_states": (_i, [_vp] * 4 + [_fp, _fp, _vp, _vp, _sz, _vp, _sz] + [_i] * 6 + [_i, _i, _i, _i, _vp]),
    "mlstm_b200_chunkwise_summary": (_i, [_vp] * 4 + [_fp] * 4 + [_vp, _sz] + [_i] * 6 + [_i, _i, _i, _i, _vp]),
    "mlstm_b200_set_unit_split": (_i, [_i]),
    "mlstm_b200_nvtx_enable": (_i, [_i]),
    "mlstm_b200_state_combine": (_i, [_fp] * 10 + [_i] * 5 + [_vp]),
    "mlstm_b200_chunkwise_dc_summary": (_i, [_vp, _vp, _fp, _vp, _sz, _fp, _vp, _sz] + [_i] * 6 + [_i, _i, _i, _f, _vp]),
    "mlstm_b200_step": (_i, [_vp] * 12 + [_i] * 7 + [_f, _vp]),
    "mlstm_b200_step_sequence": (_i, [_vp] * 12 + [_i] * 7 + [_f, _vp]),
}

_lib = None


def load():
    """Load the shared library (once).  Raises RuntimeError when it has not been built."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise RuntimeError(
            f"{LIB_PATH} is missing: build it with `python -m mlstm_kernels_b200.build` "
            "(needs nvcc; there is no CPU or PyTorch fallback for these kernels)")
    lib = C.CDLL(LIB_PATH)
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)  # AttributeError if a declared symbol is not exported
        fn.restype = res
        fn.argtypes = args
    _lib = lib
    return lib


def dtype_code(dt: torch.dtype) -> int:
    try:
        return _DTYPE_CODE[dt]
    except KeyError:
        raise ValueError(f"Unsupported kernel dtype {dt}.") from None


def code_dtype(code: int) -> torch.dtype:
    return _CODE_DTYPE[code]


def ptr(t: torch.Tensor | None):
    return None if t is None else C.c_void_p(t.data_ptr())


def stream_handle(device: torch.device):
    return C.c_void_p(torch.cuda.current_stream(device).cuda_stream)


def check(rc: int, what: str):
    if rc == 0:
        return
    lib = load()
    msg = lib.mlstm_b200_error_string(rc).decode()
    if rc == -6:
        msg += ": " + lib.mlstm_b200_last_cuda_error().decode()
        raise RuntimeError(f"{what}: {msg}")
    raise ValueError(f"{what}: {msg}")


def require_cuda(*tensors: torch.Tensor):
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise RuntimeError("mlstm_kernels_b200 kernels run on CUDA tensors only (there is no CPU fallback)")


def launch_count() -> int:
    return int(load().mlstm_b200_launch_count())


def profile_enable(on: bool = True):
    check(load().mlstm_b200_profile_enable(1 if on else 0), "mlstm_b200_profile_enable")


def profile_read() -> dict:
    """{phase name: (total milliseconds, occurrences)} since the last read; synchronises on the events."""
    lib = load()
    n = lib.mlstm_b200_profile_phases()
    ms = (C.c_float * n)()
    cnt = (C.c_int * n)()
    check(lib.mlstm_b200_profile_read(ms, cnt), "mlstm_b200_profile_read")
    return {lib.mlstm_b200_profile_phase_name(p).decode(): (float(ms[p]), int(cnt[p])) for p in range(n)}


def device_status(reset: bool = True) -> int:
    """Synchronise and return the status word of the tcgen05 kernels (0 = no bounded wait ran out)."""
    rc = int(load().mlstm_b200_device_status(1 if reset else 0))
    if rc < 0:
        check(rc, "mlstm_b200_device_status")
    return rc
