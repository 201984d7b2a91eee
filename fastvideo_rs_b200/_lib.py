"""ctypes loader for libfvsdpa.so.  There is no fallback: if the shared library is missing or a
call fails, an exception says so."""
from __future__ import annotations

import ctypes
from pathlib import Path

_PKG = Path(__file__).resolve().parent
LIB_PATH = _PKG / "libfvsdpa.so"

RAN, DECLINED = 0, 1
ERR_INVALID, ERR_CUDA, ERR_NO_DEVICE, ERR_DEVICE_STATUS, ERR_NCCL = -1, -2, -3, -4, -5


class FvError(RuntimeError):
    """A hard error from the library (negative return code)."""

    def __init__(self, code: int, text: str):
        super().__init__(f"libfvsdpa error {code}: {text}")
        self.code = code


class Declined(RuntimeError):
    """The call is outside what the kernels run (the reference's Ok(false) / Ok(None)): nothing
    was launched and there is no fallback in this package."""


class Probe(ctypes.Structure):
    _fields_ = [("backend", ctypes.c_int), ("sp_world", ctypes.c_int), ("mma_default", ctypes.c_int),
                ("has_sage", ctypes.c_int), ("sage_min_seq", ctypes.c_int), ("fp8_dense", ctypes.c_int),
                ("causal_flash", ctypes.c_int), ("kernel_choice", ctypes.c_char * 32), ("has_sm", ctypes.c_int),
                ("sm_major", ctypes.c_int), ("sms", ctypes.c_int), ("dc_loaded", ctypes.c_int),
                ("b200_loaded", ctypes.c_int), ("auto_timed", ctypes.c_int), ("cudnn_has_plan", ctypes.c_int)]


class Step(ctypes.Structure):
    _fields_ = [("kind", ctypes.c_int), ("out_bf16", ctypes.c_int), ("retired", ctypes.c_int)]


class PlanC(ctypes.Structure):
    _fields_ = [("kind", ctypes.c_int), ("has_scale", ctypes.c_int), ("scale", ctypes.c_float),
                ("has_mask", ctypes.c_int), ("fp8_first", ctypes.c_int), ("block_tokens", ctypes.c_int),
                ("window", ctypes.c_int), ("sink", ctypes.c_int), ("kv_flash", ctypes.c_int)]


_lib = None


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        if not LIB_PATH.exists():
            raise FileNotFoundError(
                f"{LIB_PATH} is missing: build it with `python -m fastvideo_rs_b200._build` (needs nvcc). "
                "This package has no CPU or PyTorch fallback.")
        _lib = ctypes.CDLL(str(LIB_PATH))
        _lib.fv_last_error.restype = ctypes.c_char_p
        _lib.fv_version.restype = ctypes.c_char_p
        _lib.fv_last_kernel.restype = ctypes.c_char_p
        _lib.fv_selftest_wait_timeout.argtypes = [ctypes.c_void_p, ctypes.c_longlong]
        for name in ("fv_probe_live", "fv_probe_default", "fv_shard_ranges", "fv_rule_shape_of"):
            getattr(_lib, name).restype = None
    return _lib


def check(rc: int, what: str) -> None:
    """Raise on anything but FV_RAN."""
    if rc == RAN:
        return
    if rc == DECLINED:
        raise Declined(f"{what}: declined (unsupported shape, dtype or device); no fallback exists here")
    raise FvError(rc, lib().fv_last_error().decode())


def last_error() -> str:
    return lib().fv_last_error().decode()


def last_kernel() -> str:
    """One line naming the kernel this thread's last successful call launched."""
    return lib().fv_last_kernel().decode()
