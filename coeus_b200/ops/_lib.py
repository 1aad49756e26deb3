"""ctypes binding of ``libcoeus_kernels.so`` (the hand-written sm_100a kernels).

The library is built in-tree by :mod:`coeus_b200.build` and loaded lazily.  An op that is
given CUDA tensors and cannot find the library raises: there is no silent fallback to a
PyTorch implementation on a GPU box.
"""
from __future__ import annotations

import ctypes
import os
import threading
from typing import Optional

import torch

from ..build import build_kernels, kernels_lib_path

_lock = threading.Lock()
_lib: Optional[ctypes.CDLL] = None


class KernelLibraryError(RuntimeError):
    pass


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        with _lock:
            if _lib is None:
                path = kernels_lib_path()
                if not path.exists():
                    try:
                        build_kernels()
                    except Exception as e:  # pragma: no cover - depends on toolchain
                        raise KernelLibraryError(
                            f"CUDA kernel library {path} is missing and could not be built: {e}"
                        ) from e
                _lib = ctypes.CDLL(str(path))
    return _traced if _traced is not None else _lib


class _TracedLib:
    """The kernel library with an NVTX range around every ``cb_*`` call, named after the entry
    point, so that a timeline shows each op of a step (host-side launch ranges; off unless
    ``COEUS_NVTX=1`` or :func:`set_op_ranges`)."""

    def __init__(self, get_cdll, push, pop) -> None:
        self._get, self._push, self._pop = get_cdll, push, pop

    def __getattr__(self, name: str):
        fn = getattr(self._get(), name)
        if not name.startswith("cb_"):
            return fn
        push, pop = self._push, self._pop

        def traced(*args):
            push(name)
            try:
                return fn(*args)
            finally:
                pop()
        self.__dict__[name] = traced        # resolved once per entry point
        return traced


_traced: Optional[_TracedLib] = None


def set_op_ranges(on: bool, push=None, pop=None) -> None:
    """Turn the per-op NVTX ranges on or off.  ``push(name)`` / ``pop()`` default to
    ``torch.cuda.nvtx.range_push`` / ``range_pop`` (tests pass recorders)."""
    global _traced
    if not on:
        _traced = None
        return

    def cdll():
        global _traced
        keep, _traced = _traced, None       # lib() must hand out the real library here
        try:
            return lib()
        finally:
            _traced = keep
    _traced = _TracedLib(cdll, push or torch.cuda.nvtx.range_push, pop or torch.cuda.nvtx.range_pop)


if os.environ.get("COEUS_NVTX") == "1" and torch.cuda.is_available():
    set_op_ranges(True)


def ptr(t: Optional[torch.Tensor]) -> ctypes.c_void_p:
    if t is None:
        return ctypes.c_void_p(0)
    return ctypes.c_void_p(t.data_ptr())


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)
_raw_device = getattr(torch._C, "_cuda_getDevice", None)


def stream_ptr() -> ctypes.c_void_p:
    """The current CUDA stream of the current device as a raw handle.  Asked of the runtime
    binding directly: ``torch.cuda.current_stream()`` builds a Python stream object through
    several layers of device-index resolution, which was a third of the host time of a training
    step (one call per kernel launch)."""
    if _raw_stream is not None and _raw_device is not None:
        return ctypes.c_void_p(_raw_stream(_raw_device()))
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


_status_bufs: dict = {}


def status_buffer(device: torch.device) -> torch.Tensor:
    """Per-device int32[4] word that kernels write a status code into (0 = ok)."""
    key = device.index if device.index is not None else torch.cuda.current_device()
    buf = _status_bufs.get(key)
    if buf is None:
        buf = torch.zeros(4, dtype=torch.int32, device=torch.device("cuda", key))
        _status_bufs[key] = buf
    return buf


def check_status(device: Optional[torch.device] = None) -> None:
    """Synchronise and raise if any kernel recorded a non-zero status since the last check."""
    from ..foundation.error import DeviceError, CommError

    device = device or torch.device("cuda", torch.cuda.current_device())
    buf = status_buffer(device)
    code, where = buf[:2].tolist()
    if code != 0:
        buf.zero_()
        if code == 4:
            raise CommError.timeout(peer=where)
        raise DeviceError.from_status(code, where)


launch_count = 0  # number of kernel launches issued through this module


def check_rc(rc: int, name: str, launches: int = 1) -> None:
    """Raise on a non-zero host-side return code; count the launches the call made."""
    global launch_count
    if rc != 0:
        raise KernelLibraryError(f"{name} failed on the host side with code {rc}")
    launch_count += launches
