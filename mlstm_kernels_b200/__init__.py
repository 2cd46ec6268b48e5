"""B200-native (sm_100a) kernels for the mLSTM hot path: chunkwise forward / backward for the
exponential and sigmoid input gate, and the recurrent decode step, behind the PyTorch-facing
interface of NX-AI/mlstm_kernels.  All compute runs in hand-written CUDA loaded from
libmlstm_b200.so through its C ABI (include/mlstm_b200.h); there is no CPU or PyTorch fallback."""

from .chunkwise import (
    chunkwise_bw_raw,
    chunkwise_fw_raw,
    chunkwise_states_raw,
    kernel_chunk_size,
    mlstm_chunkwise__b200_xl_chunk,
    resolve_chunk_size,
    mlstm_siging_chunkwise__b200_xl_chunk,
    select_chunk_size,
    tcgen05_applies,
)
from .recurrent import (
    mlstm_recurrent_sequence__b200,
    mlstm_recurrent_step__b200,
    mlstm_recurrent_step__b200_fw,
)
from .registry import get_kernel, register_with_mlstm_kernels

__all__ = [
    "mlstm_chunkwise__b200_xl_chunk",
    "mlstm_siging_chunkwise__b200_xl_chunk",
    "mlstm_recurrent_step__b200",
    "mlstm_recurrent_step__b200_fw",
    "mlstm_recurrent_sequence__b200",
    "chunkwise_fw_raw",
    "chunkwise_bw_raw",
    "chunkwise_states_raw",
    "select_chunk_size",
    "kernel_chunk_size",
    "tcgen05_applies",
    "resolve_chunk_size",
    "get_kernel",
    "register_with_mlstm_kernels",
]
