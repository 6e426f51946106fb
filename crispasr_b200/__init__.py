"""crispasr_b200 — host-side mirror of the B200 attention path behind GGML_OP_FLASH_ATTN_EXT.

The package is a thin ctypes binding over ``libb200_fattn.so`` (the C-ABI of
``include/b200_fattn.h``).  There is no CPU or PyTorch fallback: if the shared library has not
been built, importing :func:`lib` raises.
"""
from __future__ import annotations

import ctypes as C
import os

from . import abi

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libb200_fattn.so")
_LIB = None


class B200Error(RuntimeError):
    def __init__(self, code: int, where: str):
        self.code = code
        msg = lib().b200_strerror(code).decode()
        if code == abi.E_CUDA:
            msg += ": " + lib().b200_last_cuda_error().decode()
        super().__init__(f"{where}: {msg} (code {code})")


def lib() -> C.CDLL:
    """The loaded C-ABI library. Raises if it has not been built (python -m crispasr_b200.build)."""
    global _LIB
    if _LIB is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError(
                f"{LIB_PATH} is missing: build it with `python -m crispasr_b200.build` "
                "(there is no fallback implementation)")
        _LIB = abi.bind(C.CDLL(LIB_PATH))
    return _LIB


from .op import (flash_attn_ext, flash_attn_ext_host, plan, supports, workspace_bytes, KvCache,  # noqa: E402
                 SegmentScheduler)

__all__ = ["abi", "lib", "B200Error", "flash_attn_ext", "flash_attn_ext_host", "plan", "supports",
           "workspace_bytes", "KvCache", "SegmentScheduler", "LIB_PATH"]
