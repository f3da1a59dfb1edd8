"""ctypes loader of libhipster_b200.so. Fails loudly when the CUDA library is missing: there is no CPU fallback."""
import ctypes
import os
import re

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.environ.get("HIPSTER_B200_LIB") or os.path.join(HERE, "libhipster_b200.so")
HEADER = os.path.join(HERE, "..", "include", "hipster_b200.h")

_lib = None


class HipsterError(RuntimeError):
    """Raised for every non-zero status of the C ABI (the reference throws std::runtime_error, qwen35.cpp:10)."""

    def __init__(self, code, msg):
        super().__init__(f"hipster_b200 error {code}: {msg}")
        self.code = code


def declared_symbols():
    """Names of the functions declared in include/hipster_b200.h."""
    text = open(HEADER).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(hp_[a-z0-9_]+)\s*\(", text)))


def lib():
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise HipsterError(-1, f"{LIB_PATH} is missing: build it with `python -m hipster_b200.build` (needs nvcc); no fallback path exists")
        _lib = ctypes.CDLL(LIB_PATH)
        _lib.hp_last_error.restype = ctypes.c_char_p
        for name in ("hp_xq8_q_bytes", "hp_xq8_sc_bytes", "hp_argmax_scratch_bytes"):
            getattr(_lib, name).restype = ctypes.c_size_t
    return _lib


def check(code):
    if code != 0:
        raise HipsterError(code, lib().hp_last_error().decode())
    return code


def ptr(t):
    """Device (or host) pointer of a torch tensor / numpy array as c_void_p; None -> NULL."""
    if t is None:
        return ctypes.c_void_p(0)
    if hasattr(t, "data_ptr"):
        return ctypes.c_void_p(t.data_ptr())
    return ctypes.c_void_p(t.ctypes.data)
