"""ml_framework_b200: a Blackwell (sm_100a) training and serving framework.

PyTorch is the tensor/autograd layer; the hot operators are hand-written CUDA kernels
(tcgen05 / TMEM / TMA) in ``csrc/`` reached through a C ABI, and multi-GPU paths run one
process per GPU over ``torch.distributed`` with peer-mapped symmetric memory for the fused
compute+collective kernels.
"""
__version__ = "0.1.0"

import os as _os

# Kernels of the native library wait on one another across GPUs (device barriers, gathered chunks). With lazy module
# loading the first launch of a kernel may have to synchronise the context while such a wait is in progress, so all
# modules are loaded when the library is (effective when set before the CUDA context exists; an explicit setting wins).
_os.environ.setdefault("CUDA_MODULE_LOADING", "EAGER")

from . import _lib  # noqa: F401


def native_available() -> bool:
    """True when ``libmlfb200.so`` is built (or can be built) and loads."""
    return _lib.available()
