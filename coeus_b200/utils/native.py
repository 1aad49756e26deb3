"""Loader of the native host module ``_coeus_host`` (built in-tree by :mod:`coeus_b200.build`
from ``csrc/host``): tokenizers, checkpoint IO, data pipeline, text algorithms, CPU oracle."""
from __future__ import annotations

import importlib.util
import sys
import threading

from ..build import build_host, host_lib_path

_lock = threading.Lock()
_mod = None


def module():
    global _mod
    if _mod is None:
        with _lock:
            if _mod is None:
                path = host_lib_path()
                if not path.exists():
                    build_host()
                spec = importlib.util.spec_from_file_location("_coeus_host", str(path))
                mod = importlib.util.module_from_spec(spec)
                spec.loader.exec_module(mod)
                sys.modules["_coeus_host"] = mod
                _mod = mod
    return _mod


def available() -> bool:
    try:
        module()
        return True
    except Exception:
        return False


def suffix_array(text: str):
    return list(module().suffix_array(text))
