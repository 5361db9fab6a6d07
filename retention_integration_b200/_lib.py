"""ctypes binding of libpr_b200.so.

The library is the only compute path of this package: if it is missing the import
of any op fails with an error naming the build command.  Nothing here falls back
to PyTorch or CPU code.
"""
from __future__ import annotations

import ctypes
import os

PKG_DIR = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(PKG_DIR, "libpr_b200.so")

PR_BF16, PR_FP16 = 0, 1
PR_OK = 0

_lib = None


class PRError(RuntimeError):
    """A call into libpr_b200.so returned a negative status."""


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise PRError(
                f"{LIB_PATH} is missing: build it with `python -m retention_integration_b200.build` "
                "(there is no fallback path)"
            )
        _lib = ctypes.CDLL(LIB_PATH)
        _lib.pr_last_error.restype = ctypes.c_char_p
        _lib.pr_abi_version.restype = ctypes.c_int
    return _lib


def check(rc: int, what: str) -> None:
    if rc != PR_OK:
        msg = lib().pr_last_error().decode("utf-8", "replace")
        raise PRError(f"{what} failed with code {rc}: {msg}")


def dtype_code(dtype) -> int:
    import torch

    if dtype == torch.bfloat16:
        return PR_BF16
    if dtype == torch.float16:
        return PR_FP16
    raise PRError(f"unsupported dtype {dtype}: the kernels take bfloat16 or float16")


def ptr(t) -> ctypes.c_void_p:
    """Device pointer of a tensor (None -> NULL)."""
    return ctypes.c_void_p(0 if t is None else t.data_ptr())


def stream_ptr(device) -> ctypes.c_void_p:
    import torch

    return ctypes.c_void_p(torch.cuda.current_stream(device).cuda_stream)


def device_status(device_index: int) -> int:
    """Synchronise-free read of the status word; call after a synchronize."""
    out = ctypes.c_int(0)
    check(lib().pr_device_status(ctypes.c_int(device_index), ctypes.byref(out)), "pr_device_status")
    return out.value
