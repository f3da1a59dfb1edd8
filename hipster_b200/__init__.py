"""hipster_b200: B200-native MTP speculative-decode path behind the reference's engine/kernel interface.

Python here is only the host-side mirror of the reference interface (engine/kernels/gemv.h, ops.h and the
engine classes) over the C ABI of libhipster_b200.so; torch is used for device memory and streams.
"""
from ._lib import HipsterError, lib, check, ptr, declared_symbols, LIB_PATH  # noqa: F401
from . import kernels  # noqa: F401
from .engine import Engine, ModelCfg, SlotReq  # noqa: F401
