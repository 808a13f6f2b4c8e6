"""sanic_b200 — B200 (sm_100a) backend for sanic's derived carriers.

Everything computes through libsanic_b200.so (see include/sanic_b200.h). The package has no
CPU fallback: `CudaDevice()` raises without a CUDA device, and `_abi.load()` raises if the
library has not been built.
"""
from . import _abi as abi  # noqa: F401
from .backend import (CompileError, CudaDevice, RunError, carrier_contraction, carrier_deferred_norm,  # noqa: F401
                      carrier_extremum_index, carrier_online_softmax, make_carrier)

__all__ = ["abi", "CudaDevice", "CompileError", "RunError", "make_carrier", "carrier_online_softmax",
           "carrier_deferred_norm", "carrier_contraction", "carrier_extremum_index"]
