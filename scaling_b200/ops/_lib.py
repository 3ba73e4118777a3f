"""ctypes loader for ``libsb200.so`` (the sm_100a kernels of scaling_b200).

``lib()`` returns the loaded library, building it first when the sources changed and nvcc is
available.  On a machine with a GPU a missing library is an error: the CUDA kernels are the
product, the torch expressions in ``scaling_b200.ops`` exist for CPU ranks and as test oracles.
"""

from __future__ import annotations

import ctypes
import os
import threading
from ctypes import c_float, c_int, c_long, c_void_p
from typing import Optional

import torch

from . import _build

_LIB: Optional["_Counting"] = None
_LOCK = threading.Lock()

SB_OK = 0
SB_ERR_WAIT_TIMEOUT = 101
SB_ERR_BAD_ARG = 102
SB_ERR_TOO_LARGE = 103
SB_ERR_DRIVER = 104

_ERR_NAMES = {
    SB_ERR_WAIT_TIMEOUT: "a bounded device-side wait timed out",
    SB_ERR_BAD_ARG: "bad argument (shape / alignment / dtype not supported by the kernel)",
    SB_ERR_TOO_LARGE: "size exceeds a static limit of the kernel",
    SB_ERR_DRIVER: "CUDA driver entry point or tensor-map encode failed",
}


class KernelError(RuntimeError):
    pass


class CommTimeout(KernelError):
    """A device-side wait on a peer flag or barrier gave up; the CUDA context is still usable."""


def check(rc: int, what: str) -> None:
    if rc == SB_OK:
        return
    if rc == SB_ERR_WAIT_TIMEOUT:
        raise CommTimeout(f"{what}: {_ERR_NAMES[rc]}")
    if rc in _ERR_NAMES:
        raise KernelError(f"{what}: {_ERR_NAMES[rc]}")
    raise KernelError(f"{what}: CUDA error {rc}")


_SIGS = {
    # name: argtypes (restype is always int unless listed in _RESTYPES)
    "sb200_norm_fwd": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_float, c_int, c_int, c_void_p],
    "sb200_norm_bwd_partial_rows": [c_int, c_int],
    "sb200_norm_bwd_partial_rows_h": [c_int, c_int, c_int, c_int],
    "sb200_norm_bwd": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p],
    "sb200_swiglu_fwd": [c_void_p, c_void_p, c_void_p, c_long, c_int, c_long, c_long, c_long, c_float, c_int, c_void_p],
    "sb200_swiglu_bwd": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_long, c_int, c_long, c_long, c_long, c_long, c_long, c_float, c_int, c_void_p],
    "sb200_gelu_fwd": [c_void_p, c_void_p, c_long, c_int, c_void_p],
    "sb200_gelu_bwd_colsum": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_long, c_int, c_int, c_int, c_int, c_void_p],
    "sb200_gelu_bwd": [c_void_p, c_void_p, c_void_p, c_long, c_int, c_void_p],
    "sb200_dropout_add": [c_void_p, c_void_p, c_void_p, c_long, c_float, c_float, c_float, c_void_p, ctypes.c_uint, c_long, c_int, c_int, c_void_p],
    "sb200_rope": [c_void_p, c_void_p, c_int, c_int, c_int, c_long, c_long, c_float, c_int, c_int, c_int, c_void_p],
    "sb200_masked_softmax_fwd": [c_void_p, c_void_p, c_void_p, c_long, c_int, c_int, c_int, c_float, c_int, c_void_p],
    "sb200_masked_softmax_bwd": [c_void_p, c_void_p, c_void_p, c_void_p, c_long, c_int, c_int, c_int, c_float, c_int, c_void_p],
    "sb200_colsum_splits": [c_long, c_int, c_int, c_int],
    "sb200_colsum": [c_void_p, c_void_p, c_void_p, c_long, c_int, c_long, c_int, c_int, c_int, c_void_p],
    "sb200_transpose": [c_void_p, c_void_p, c_int, c_int, c_int, c_void_p],
    "sb200_ce_stats": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_long, c_int, c_long, c_long, c_int, c_void_p],
    "sb200_ce_finalize": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_long, c_int, c_long, c_long, c_long, c_void_p, c_int, c_void_p],
    "sb200_scale_by_dev": [c_void_p, c_void_p, c_float, c_long, c_int, c_void_p],
    "sb200_adamw": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_long, c_float, c_float, c_float, c_float, c_float, c_float, c_float, c_void_p, c_void_p, c_int, c_int, c_void_p],
    "sb200_sumsq_max_partials": [],
    "sb200_sumsq": [c_void_p, c_long, c_void_p, c_void_p, c_void_p, c_float, c_int, c_int, c_void_p],
    "sb200_step_control": [c_int, c_void_p, c_void_p, c_void_p, c_float, c_float, c_float, c_void_p, c_void_p, c_void_p],
    "sb200_embedding_fwd": [c_void_p, c_void_p, c_void_p, c_long, c_int, c_long, c_long, c_int, c_void_p],
    "sb200_embedding_bwd": [c_void_p, c_void_p, c_void_p, c_void_p, c_long, c_int, c_long, c_long, c_int, c_int, c_void_p],
    "sb200_p2p_max_ranks": [],
    "sb200_p2p_barrier": [c_void_p, c_void_p, c_int, c_int, c_void_p, ctypes.c_double, c_void_p],
    "sb200_p2p_reduce_scatter": [c_void_p, c_void_p, c_long, c_long, c_int, c_int, c_int, c_void_p],
    "sb200_p2p_all_gather": [c_void_p, c_void_p, c_void_p, c_long, c_long, c_int, c_int, c_int, c_void_p],
    "sb200_gemm_ws": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_long, c_long, c_long, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p, c_long, c_void_p, c_void_p],
    "sb200_gemm_fp8": [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_long, c_long, c_long, c_int, c_int, c_int, c_int, c_int, c_void_p, c_long, c_void_p, c_void_p],
    "sb200_gemm": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_long, c_long, c_long, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p],
}


def available() -> bool:
    """True when the native library can be used in this process (CUDA device present)."""
    return torch.cuda.is_available()


class _Counting:
    """Proxy over the loaded library that counts calls into kernel-launching entry points."""

    def __init__(self, handle: ctypes.CDLL):
        self._handle = handle
        self.calls = 0
        self._cache: dict[str, object] = {}
        self._tls = threading.local()

    def _bind_thread(self) -> None:
        """First call from a host thread: select torch's current device in the library's own CUDA runtime."""
        dev = torch.cuda.current_device()
        if getattr(self._tls, "device", None) != dev:
            rc = self._handle.sb200_bind_device(int(dev))
            if rc != 0:
                raise KernelError(f"sb200_bind_device({dev}) failed with CUDA error {rc}")
            self._tls.device = dev

    def __getattr__(self, name: str):
        fn = self._cache.get(name)
        if fn is None:
            raw = getattr(self._handle, name)
            if name in _NO_LAUNCH:
                fn = raw
            else:
                def fn(*args, _raw=raw, _self=self):
                    _self._bind_thread()
                    _self.calls += 1
                    return _raw(*args)
            self._cache[name] = fn
        return fn

    def has(self, name: str) -> bool:
        return hasattr(self._handle, name)


_NO_LAUNCH = {"sb200_p2p_max_ranks", "sb200_colsum_splits", "sb200_norm_bwd_partial_rows", "sb200_norm_bwd_partial_rows_h", "sb200_sumsq_max_partials",
              "sb200_bind_device", "sb200_fa_last_driver_error"}


def kernel_calls() -> int:
    """Number of calls made so far into kernel-launching entry points of the native library."""
    return 0 if _LIB is None else _LIB.calls


def note_replayed_calls(n: int) -> None:
    """Account for ``n`` kernel-launching calls that a CUDA-graph replay repeated on the device."""
    if _LIB is not None:
        _LIB.calls += int(n)


def lib() -> "_Counting":
    global _LIB
    if _LIB is not None:
        return _LIB
    with _LOCK:
        if _LIB is not None:
            return _LIB
        path = _build.LIB_PATH
        if not path.exists() or (os.environ.get("SB200_AUTOBUILD", "1") == "1" and _can_build() and _build.needs_build()):
            if not _can_build():
                raise KernelError(
                    f"{path} is missing and nvcc is not available; run `python -m scaling_b200.ops._build` "
                    "on a machine with the CUDA toolkit"
                )
            _build.build()
        handle = ctypes.CDLL(str(path))
        for name, argtypes in _SIGS.items():
            if hasattr(handle, name):
                fn = getattr(handle, name)
                fn.argtypes = argtypes
                fn.restype = c_int
        _LIB = _Counting(handle)
        return _LIB


def lib_has(name: str) -> bool:
    """True when a GPU is present and the loaded library exports ``name``."""
    return available() and lib().has(name)


def declare(name: str, argtypes: list, restype=c_int):
    """Declare the signature of an exported symbol that is not in the static table."""
    fn = getattr(lib()._handle, name)
    fn.argtypes = argtypes
    fn.restype = restype
    return fn


def _can_build() -> bool:
    try:
        _build._nvcc()
        return True
    except RuntimeError:
        return False


_DT = {torch.float32: 0, torch.bfloat16: 1, torch.float16: 2}


def dt(t: torch.dtype) -> int:
    try:
        return _DT[t]
    except KeyError:
        raise KernelError(f"dtype {t} is not supported by the sm_100a kernels") from None


def ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


def stream() -> int:
    return torch.cuda.current_stream().cuda_stream


_SM_COUNT: dict[int, int] = {}


def sm_count() -> int:
    d = torch.cuda.current_device()
    if d not in _SM_COUNT:
        _SM_COUNT[d] = torch.cuda.get_device_properties(d).multi_processor_count
    return _SM_COUNT[d]
