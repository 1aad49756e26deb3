"""ctypes binding of ``libcoeus_kernels.so`` (the hand-written sm_100a kernels).

The library is built in-tree by :mod:`coeus_b200.build` and loaded lazily.  An op that is
given CUDA tensors and cannot find the library raises: there is no silent fallback to a
PyTorch implementation on a GPU box.
"""
from __future__ import annotations

import ctypes
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
    return _lib


def ptr(t: Optional[torch.Tensor]) -> ctypes.c_void_p:
    if t is None:
        return ctypes.c_void_p(0)
    return ctypes.c_void_p(t.data_ptr())


def stream_ptr() -> ctypes.c_void_p:
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
