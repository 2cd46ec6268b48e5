"""Registration of the B200 kernels with the reference package's kernel registries.

The reference resolves kernels by name from module-level dicts
(mlstm_kernels/torch/__init__.py:35-120; dicts in torch/chunkwise/__init__.py:9-15 and
torch/recurrent/__init__.py:13-24).  `register_with_mlstm_kernels()` inserts the kernels of this
package so that

    mLSTMBackendConfig(chunkwise_kernel="chunkwise--b200_xl_chunk", step_kernel="b200",
                       sequence_kernel="native_sequence__b200")

selects them, without editing the reference.  The sigmoid-gate entry contains "siging" in its name
because mLSTMBackend forwards `normalize` only to kernels so named (backend_module.py:198-199).
"""

from __future__ import annotations

from .chunkwise import mlstm_chunkwise__b200_xl_chunk, mlstm_siging_chunkwise__b200_xl_chunk
from .recurrent import mlstm_recurrent_sequence__b200, mlstm_recurrent_step__b200

CHUNKWISE_KERNELS = {
    "b200_xl_chunk": mlstm_chunkwise__b200_xl_chunk,
    "b200_xl_chunk_siging": mlstm_siging_chunkwise__b200_xl_chunk,
}
STEP_KERNELS = {"b200": mlstm_recurrent_step__b200}
SEQUENCE_KERNELS = {"native_sequence__b200": mlstm_recurrent_sequence__b200}


def get_kernel(name: str):
    """Resolve "chunkwise--b200_xl_chunk"-style names the way the reference's get_mlstm_kernel does."""
    module_type, _, kernel_name = name.partition("--")
    table = {"chunkwise": CHUNKWISE_KERNELS}.get(module_type)
    if table is None or kernel_name not in table:
        raise ValueError(f"Unknown mlstm kernel name: {name}. Available: "
                         + ", ".join(f"chunkwise--{k}" for k in CHUNKWISE_KERNELS))
    return table[kernel_name]


def register_with_mlstm_kernels() -> bool:
    """Insert this package's kernels into the registries of an importable `mlstm_kernels`.
    Returns False when that package is not installed."""
    try:
        import mlstm_kernels.torch.chunkwise as ref_cw
        import mlstm_kernels.torch.recurrent as ref_rec
    except ImportError:
        return False
    ref_cw.registry.update(CHUNKWISE_KERNELS)
    ref_rec.registry_step.update(STEP_KERNELS)
    ref_rec.registry_sequence.update(SEQUENCE_KERNELS)
    return True
