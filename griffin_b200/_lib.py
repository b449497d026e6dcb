"""ctypes binding of librglru_b200.so (the C ABI declared in include/rglru_b200.h).

There is no fallback: if the shared library is missing or a call fails, an
exception is raised.  Error classes follow the reference's conventions for this
path (griffin/triton_scan.py:213-224): RuntimeError for a missing runtime or a
failed launch, ValueError for shapes, TypeError for dtypes.
"""

from __future__ import annotations

import ctypes
import os
import threading

_PKG_DIR = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_PKG_DIR, "librglru_b200.so")

F32, BF16 = 0, 1
TOK_CUT_MASK, TOK_RESET, TOK_INACTIVE, TOK_ZERO_HISTORY = 0x03, 0x04, 0x08, 0x10

(OK, ERR_NULL_POINTER, ERR_BAD_DTYPE, ERR_BAD_SHAPE, ERR_MISALIGNED, ERR_WORKSPACE, ERR_LAUNCH,
 ERR_DEVICE_TIMEOUT, ERR_UNSUPPORTED, ERR_TOO_LARGE) = range(10)

_vp, _sz, _i, _f = ctypes.c_void_p, ctypes.c_size_t, ctypes.c_int, ctypes.c_float

# name -> (restype, argtypes); mirrors include/rglru_b200.h one to one.
SIGNATURES = {
    "rglru_status_string": (ctypes.c_char_p, [_i]),
    "rglru_last_cuda_error": (ctypes.c_char_p, []),
    "rglru_abi_version": (_i, []),
    "rglru_device_status": (_i, [ctypes.POINTER(_i)]),
    "rglru_selftest_wait_timeout": (_i, [ctypes.c_uint, _vp, _vp]),
    "rglru_chunk_steps": (_i, [_i]),
    "rglru_workspace_bytes": (_sz, [_i, _i, _i, _i]),
    "rglru_fwd": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _sz, _i, _i, _i, _f, _i, _vp]),
    "rglru_fwd_carry": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _sz, _i, _i, _i, _f, _i, _vp]),
    "rglru_bwd": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _sz, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _f, _i, _vp]),
    "rglru_conv_scan_fwd": (_i, [_vp] * 11 + [_vp, _sz, _i, _i, _i, _f, _i, _vp]),
    "rglru_conv_scan_bwd": (_i, [_vp] * 11 + [_vp, _sz] + [_vp] * 5 + [_i, _i, _i, _f, _i, _vp]),
    "rglru_merge_fwd": (_i, [_vp] * 12 + [_vp, _sz, _i, _i, _i, _f, _i, _vp]),
    "rglru_merge_bwd": (_i, [_vp] * 12 + [_vp, _sz] + [_vp] * 6 + [_i, _i, _i, _f, _i, _vp]),
    "rglru_grouped_fwd": (_i, [_vp] * 9 + [_vp, _sz, _i, _i, _i, _i, _f, _i, _vp]),
    "rglru_grouped_bwd": (_i, [_vp] * 9 + [_vp, _sz] + [_vp] * 6 + [_i, _i, _i, _i, _f, _i, _vp]),
    "rglru_linear_scan_fwd": (_i, [_vp, _vp, _vp, _vp, _i, _i, _i, _vp]),
    "rglru_linear_scan_bwd": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _vp]),
    "rglru_conv_fwd": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _vp]),
    "rglru_conv_bwd_workspace_bytes": (_sz, [_i, _i, _i]),
    "rglru_conv_bwd": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _sz, _i, _i, _i, _i, _vp]),
    "rglru_conv_bwd_noalloc_max_bytes": (_sz, []),
    "rglru_conv_bwd_noalloc": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _vp]),
    "rglru_column_sums_workspace_bytes": (_sz, [ctypes.c_longlong, _i]),
    "rglru_column_sums": (_i, [_vp, _vp, _vp, _sz, ctypes.c_longlong, _i, _i, _vp]),
    "rglru_decode_conv": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _vp]),
    "rglru_decode_step": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _f, _i, _vp]),
}

_lock = threading.Lock()
_lib = None


def load() -> ctypes.CDLL:
    """Load the library once; raise RuntimeError if it has not been built."""
    global _lib
    with _lock:
        if _lib is None:
            if not os.path.exists(LIB_PATH):
                raise RuntimeError(
                    f"CUDA RG-LRU library not found at {LIB_PATH}; build it with `python -m griffin_b200.build`. "
                    "scan_mode='cuda' has no CPU or Triton fallback."
                )
            lib = ctypes.CDLL(LIB_PATH)
            for name, (restype, argtypes) in SIGNATURES.items():
                fn = getattr(lib, name)
                fn.restype = restype
                fn.argtypes = argtypes
            _lib = lib
        return _lib


def status_text(code: int) -> str:
    return load().rglru_status_string(code).decode()


def check(code: int, what: str) -> None:
    """Turn a non-zero status into the exception class the reference would raise."""
    if code == OK:
        return
    lib = load()
    text = f"{what}: {lib.rglru_status_string(code).decode()}"
    if code in (ERR_BAD_SHAPE, ERR_NULL_POINTER, ERR_MISALIGNED, ERR_WORKSPACE, ERR_TOO_LARGE):
        raise ValueError(text)
    if code == ERR_BAD_DTYPE:
        raise TypeError(text)
    if code == ERR_LAUNCH:
        text += f" ({lib.rglru_last_cuda_error().decode()})"
    raise RuntimeError("CUDA RG-LRU " + text)


_TIMEOUT_NAMES = {1: "a tile load never completed", 2: "the producer never saw a chunk's results",
                  3: "the wait self-test gave up (as it must)"}


def check_device() -> None:
    """Synchronise the current device and raise RuntimeError if a bounded wait inside a kernel has expired since
    the last check (the kernel then ran to its end on garbage: its outputs, and gradients computed from them,
    must not be used).  The check costs a device synchronisation, so it belongs at step boundaries -- a
    training loop can call it every N optimizer steps; nothing on the operator path calls it by itself."""
    detail = _i(0)
    rc = load().rglru_device_status(ctypes.byref(detail))
    if rc == ERR_DEVICE_TIMEOUT:
        raise RuntimeError(f"CUDA RG-LRU: a bounded wait inside a kernel expired (detail {detail.value}: "
                           f"{_TIMEOUT_NAMES.get(detail.value, 'unknown')}); results since the last check are invalid")
    check(rc, "rglru_device_status")


def device_status() -> int:
    """Synchronise and return the device status word (0 = no bounded wait expired)."""
    detail = _i(0)
    load().rglru_device_status(ctypes.byref(detail))
    return detail.value
