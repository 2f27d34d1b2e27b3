"""Python face of the lean device runtime (``csrc/kernels/devrt.cu``): prioritised main + side streams
with fork/join, stream capture -> graph, pinned staging, async copies.  Kernels of the library take
the stream handle of ``stream(which)``."""
from __future__ import annotations

import ctypes
from typing import Optional

from .. import _lib


class DeviceRuntime:
    def __init__(self, device: int = 0, n_side: int = 2):
        self.K = _lib.lib()
        self.h = ctypes.c_void_p()
        self._rc(self.K.lib.fb_rt_create(ctypes.c_int64(device), ctypes.c_int64(n_side), ctypes.byref(self.h)), "create")
        self.K.lib.fb_rt_stream.restype = ctypes.c_void_p
        self.n_side = n_side

    @staticmethod
    def _rc(rc: int, what: str):
        if rc != 0:
            raise _lib.KernelError(f"fb_rt_{what} failed with CUDA error {rc}")

    def stream(self, which: int = -1) -> int:
        """CUDA stream handle: -1 = main, 0.. = side streams."""
        return int(self.K.lib.fb_rt_stream(self.h, ctypes.c_int64(which)) or 0)

    def fork(self, which: int):
        self._rc(self.K.lib.fb_rt_fork(self.h, ctypes.c_int64(which)), "fork")

    def join(self, which: int):
        self._rc(self.K.lib.fb_rt_join(self.h, ctypes.c_int64(which)), "join")

    def sync(self):
        self._rc(self.K.lib.fb_rt_sync(self.h), "sync")

    def capture_begin(self):
        self._rc(self.K.lib.fb_rt_capture_begin(self.h), "capture_begin")

    def capture_end(self) -> int:
        g = ctypes.c_void_p()
        self._rc(self.K.lib.fb_rt_capture_end(self.h, ctypes.byref(g)), "capture_end")
        return g.value

    def graph_launch(self, graph: int):
        self._rc(self.K.lib.fb_rt_graph_launch(self.h, ctypes.c_void_p(graph)), "graph_launch")

    def graph_free(self, graph: int):
        self._rc(self.K.lib.fb_rt_graph_free(ctypes.c_void_p(graph)), "graph_free")

    def copy(self, dst: int, src: int, nbytes: int, which: int = -1):
        self._rc(self.K.lib.fb_rt_copy(self.h, ctypes.c_void_p(dst), ctypes.c_void_p(src), ctypes.c_int64(nbytes),
                                       ctypes.c_int64(which)), "copy")

    def pinned_alloc(self, nbytes: int) -> int:
        p = ctypes.c_void_p()
        self._rc(self.K.lib.fb_rt_pinned_alloc(ctypes.c_int64(nbytes), ctypes.byref(p)), "pinned_alloc")
        return p.value

    def pinned_free(self, p: int):
        self._rc(self.K.lib.fb_rt_pinned_free(ctypes.c_void_p(p)), "pinned_free")

    def close(self):
        if self.h:
            self.K.lib.fb_rt_destroy(self.h)
            self.h = ctypes.c_void_p()
