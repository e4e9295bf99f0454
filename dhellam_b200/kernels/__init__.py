"""ctypes loader for the sm_100a kernel library.

``lib()`` returns the loaded ``libdhellam_b200.so``.  On a machine with a GPU a missing
or unloadable library is an error (no silent fall-back to PyTorch); on a CPU-only
machine ``available()`` is False and the ops layer uses its fp32 reference path.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import c_char_p, c_float, c_int, c_int64, c_uint64, c_void_p
from pathlib import Path

import torch

_LIB = None
_LIB_PATH = Path(__file__).resolve().parent.parent / "lib" / "libdhellam_b200.so"


class KernelError(RuntimeError):
    """A launch was refused by the library (bad arguments, failed launch)."""


class DeviceWaitTimeout(RuntimeError):
    """A bounded device-side wait gave up; the status word says where."""


class Status(ctypes.Structure):
    _fields_ = [("code", c_int), ("where", c_int), ("block", c_int), ("extra", c_int)]


def available() -> bool:
    return torch.cuda.is_available()


# Which implementation the ops layer uses for CUDA tensors: "native" = this library's sm_100a
# kernels (the product); "library" = PyTorch / cuBLAS / flash-attn calls only, never touching
# libdhellam_b200.so.  The second exists for one purpose: the labelled composition arm of the
# benchmark, which times the reference's recipe (torch.matmul, flash-attn, NCCL, eager PyTorch
# elementwise ops; dhellam/operators/*.py) on the same box.
_BACKEND = os.environ.get("DHELLAM_OPS_BACKEND", "native")


def set_backend(name: str):
    global _BACKEND
    assert name in ("native", "library"), name
    _BACKEND = name


def backend() -> str:
    return _BACKEND


def use_native(t) -> bool:
    """True when an op on tensor ``t`` should run this library's kernel."""
    return t.is_cuda and _BACKEND == "native"


def use_library(t) -> bool:
    """True when an op on CUDA tensor ``t`` should run the PyTorch / vendor-library composition."""
    return t.is_cuda and _BACKEND == "library"


# Reproducible mode: every reduction whose order would depend on timing (norm weight gradients, the embedding
# gradient, the gradient norm, K-split weight-gradient GEMMs) takes a fixed-order form, so that two runs of
# the same program on the same GPU give bitwise equal results.  Costs a few small extra launches per layer.
_DETERMINISTIC = os.environ.get("DHELLAM_DETERMINISTIC", "0") == "1"
_DET_SCRATCH = {}


def set_deterministic(on: bool = True):
    global _DETERMINISTIC
    _DETERMINISTIC = bool(on)
    if available() and _BACKEND == "native":
        proto("dh_gemm_set_splitk", [c_int], None)(1 if on else -1)


def deterministic() -> bool:
    return _DETERMINISTIC


def det_scratch(device, floats: int, zero_tail: bool = False):
    """A per-device fp32 scratch of at least ``floats`` elements for the fixed-order reductions (grown on demand;
    the users run on one stream, in order).  ``zero_tail`` scratch starts zeroed and is kept separately."""
    key = (torch.device(device).index, zero_tail)
    buf = _DET_SCRATCH.get(key)
    if buf is None or buf.numel() < floats:
        buf = (torch.zeros if zero_tail else torch.empty)(floats, dtype=torch.float32, device=device)
        _DET_SCRATCH[key] = buf
    return buf


def lib_path() -> Path:
    return _LIB_PATH


def lib():
    global _LIB
    if _BACKEND == "library":
        raise KernelError("the ops backend is 'library' (composition arm): the sm_100a kernel library must not be used")
    if _LIB is not None:
        return _LIB
    if not _LIB_PATH.exists():
        if os.environ.get("DHELLAM_B200_BUILD_ON_IMPORT", "1") == "1":
            from .build import build
            build()
        else:
            raise KernelError(f"{_LIB_PATH} is missing; run python -m dhellam_b200.kernels.build")
    _LIB = ctypes.CDLL(str(_LIB_PATH))
    _declare(_LIB)
    return _LIB


def _declare(L):
    L.dh_status_device_ptr.restype = c_void_p
    L.dh_status_read.argtypes = [ctypes.POINTER(Status), c_int]
    L.dh_last_error_string.restype = c_char_p
    L.dh_sm_count.restype = c_int
    # The remaining prototypes are attached by the modules that use them (see _proto).


def proto(name: str, argtypes, restype=c_int):
    fn = getattr(lib(), name)
    if not getattr(fn, "_dh_declared", False):
        fn.argtypes = argtypes
        fn.restype = restype
        fn._dh_declared = True
    return fn


_LAUNCHES = 0


def launch_count() -> int:
    """Number of calls into the kernel library so far (each launches at least one kernel)."""
    return _LAUNCHES


def check(rc: int, what: str = "kernel"):
    global _LAUNCHES
    _LAUNCHES += 1
    if rc != 0:
        msg = lib().dh_last_error_string().decode()
        raise KernelError(f"{what} failed (code {rc}): {msg}")


def read_status(clear: bool = True) -> Status:
    """Synchronises the device and returns the status word."""
    st = Status()
    check(lib().dh_status_read(ctypes.byref(st), 1 if clear else 0), "dh_status_read")
    return st


def raise_on_device_error():
    st = read_status(clear=True)
    if st.code != 0:
        raise DeviceWaitTimeout(f"device status code={st.code} where={st.where} block={st.block} extra={st.extra}")


def stream_ptr(stream=None) -> int:
    s = stream if stream is not None else torch.cuda.current_stream()
    return s.cuda_stream


def ptr(t) -> int:
    return 0 if t is None else t.data_ptr()
