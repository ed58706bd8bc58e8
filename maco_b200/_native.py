"""ctypes binding of ``libmaco_b200.so``.

The library is a plain shared object with ``extern "C"`` entry points (no libtorch, no libcuda
link dependency), so it loads on a machine without a GPU. On a machine WITH a GPU a missing
library is an error, not a reason to fall back to PyTorch: :func:`lib` raises.
"""
from __future__ import annotations

import ctypes
import os
import threading
from pathlib import Path
from typing import Optional

import torch

_LIB_PATH = Path(__file__).resolve().parent / "_lib" / "libmaco_b200.so"
_lock = threading.Lock()
_lib: Optional[ctypes.CDLL] = None

c_void_p, c_int, c_ll, c_float, c_double, c_uint, c_u64 = (
    ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong, ctypes.c_float, ctypes.c_double, ctypes.c_uint,
    ctypes.c_uint64,
)

DT_BF16, DT_F16, DT_F32 = 0, 1, 2
DTYPE_CODE = {torch.bfloat16: DT_BF16, torch.float16: DT_F16, torch.float32: DT_F32}

STATUS_TIMEOUT, STATUS_BAD_TASK, STATUS_QUEUE_OVERFLOW, STATUS_PEER_TIMEOUT = 1, 2, 4, 8


class NativeLibraryError(ImportError):
    pass


def _declare(lib: ctypes.CDLL) -> None:
    P, I, LL, F, D = c_void_p, c_int, c_ll, c_float, c_double
    sigs = {
        "maco_last_error": (ctypes.c_char_p, []),
        "maco_status": (c_uint, [I]),
        "maco_sm_count": (I, []),
        "maco_gemm": (I, [P, P, P, I, I, I, LL, LL, LL, I, I, I, I, I, P, I, P, LL, I, F, I, I, D, P, I]),
        "maco_gemm_tf32": (I, [P, P, P, I, I, I, LL, LL, LL, I, I, P, I, P, LL, I, F, I, D, P]),
        "maco_gemm_simt": (I, [P, P, P, I, I, I, LL, LL, LL, LL, LL, I, I, I, P, I, P, LL, I, F, P]),
    }
    for name, (res, args) in sigs.items():
        if hasattr(lib, name):
            fn = getattr(lib, name)
            fn.restype = res
            fn.argtypes = args


def declare(name: str, restype, argtypes) -> None:
    """Declares the prototype of an entry point defined outside the core table above."""
    fn = getattr(lib(), name)
    fn.restype = restype
    fn.argtypes = argtypes


def available() -> bool:
    return _LIB_PATH.exists()


def lib() -> ctypes.CDLL:
    """Returns the loaded library; builds it first if it is missing and nvcc is present."""
    global _lib
    if _lib is not None:
        return _lib
    with _lock:
        if _lib is not None:
            return _lib
        if not _LIB_PATH.exists():
            if os.environ.get("MACO_NO_AUTOBUILD", "0") != "1":
                try:
                    from . import _build
                    _build.build()
                except Exception as exc:  # pragma: no cover - depends on toolchain
                    raise NativeLibraryError(
                        f"{_LIB_PATH} is missing and building it failed: {exc}\n"
                        "Hint: run `python -m maco_b200._build` where nvcc (CUDA >= 12.8) is installed"
                    ) from exc
            if not _LIB_PATH.exists():
                raise NativeLibraryError(f"{_LIB_PATH} is missing; run `python -m maco_b200._build`")
        handle = ctypes.CDLL(str(_LIB_PATH))
        _declare(handle)
        _lib = handle
        return _lib


def last_error() -> str:
    return lib().maco_last_error().decode(errors="replace")


def check(rc: int, what: str) -> None:
    if rc != 0:
        raise RuntimeError(f"{what} failed (rc={rc}): {last_error()}")


def current_stream_ptr(stream: Optional[torch.cuda.Stream] = None) -> int:
    s = stream if stream is not None else torch.cuda.current_stream()
    return s.cuda_stream


def ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


def status(clear: bool = True) -> int:
    """OR of the failure bits kernels reported since the last clear (0 = none)."""
    return int(lib().maco_status(1 if clear else 0))
