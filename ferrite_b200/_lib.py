"""ctypes loader for the sm_100a kernel library (``libferrite_b200_kernels.so``).

The library is built in-tree by :mod:`ferrite_b200.build`.  Loading checks the build id
baked into the binary against the hash of the sources on disk and refuses a stale pair.
On a machine with a GPU the ops fail loudly when the library is missing: there is no eager
fallback behind the CUDA path.
"""
from __future__ import annotations

import ctypes
import os
from pathlib import Path
from typing import Optional

import torch

_PKG = Path(__file__).resolve().parent
_LIB_PATH = _PKG / "libferrite_b200_kernels.so"


class KernelError(RuntimeError):
    pass


class KernelLib:
    def __init__(self, path: Path = _LIB_PATH, check_build_id: bool = True):
        if not path.exists():
            raise KernelError(f"{path} is missing: run `python -m ferrite_b200.build`")
        self.path = path
        self.lib = ctypes.CDLL(str(path))
        self.lib.fb_build_id.restype = ctypes.c_char_p
        self.build_id = self.lib.fb_build_id().decode()
        if check_build_id and (_PKG.parent / "csrc" / "kernels").exists():
            from .build import kernel_build_id
            want = kernel_build_id()
            if want != self.build_id:
                raise KernelError(f"stale kernel library: built from {self.build_id}, sources are {want}; "
                                  "rebuild with `python -m ferrite_b200.build`")
        self._fns = {}
        self.launches = 0  # kernels launched through this handle (entry points, not replays)

    def fn(self, name: str):
        f = self._fns.get(name)
        if f is None:
            f = getattr(self.lib, name)
            f.restype = ctypes.c_int
            self._fns[name] = f
        return f

    def call(self, name: str, *args, stream: Optional[int] = None):
        cargs = []
        for a in args:
            if isinstance(a, torch.Tensor) or hasattr(a, "data_ptr"):
                cargs.append(ctypes.c_void_p(a.data_ptr()))
            elif a is None:
                cargs.append(ctypes.c_void_p(0))
            elif isinstance(a, bool):
                cargs.append(ctypes.c_int64(int(a)))
            elif isinstance(a, int):
                cargs.append(ctypes.c_int64(a))
            elif isinstance(a, float):
                cargs.append(ctypes.c_float(a))
            elif isinstance(a, (ctypes._SimpleCData, ctypes.Array, ctypes._Pointer)):
                cargs.append(a)
            else:
                raise TypeError(f"{name}: unsupported argument {type(a)}")
        if stream is None:
            stream = torch.cuda.current_stream().cuda_stream
        cargs.append(ctypes.c_void_p(stream))
        rc = self.fn(name)(*cargs)
        self.launches += 1
        if rc != 0:
            raise KernelError(f"{name} failed with CUDA error {rc}")


_LIB: Optional[KernelLib] = None


def lib() -> KernelLib:
    global _LIB
    if _LIB is None:
        _LIB = KernelLib()
    return _LIB


def have_lib() -> bool:
    return _LIB_PATH.exists()


def ptr(t: torch.Tensor, offset_elems: int = 0) -> ctypes.c_void_p:
    """Raw pointer into a tensor's storage, offset by elements (for column views)."""
    return ctypes.c_void_p(t.data_ptr() + offset_elems * t.element_size())
