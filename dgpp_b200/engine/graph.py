"""Native CUDA-graph executor (csrc/engine/graph_exec.cu): capture a launch sequence once, replay it with
programmatic-dependent-launch edges between the kernels.  Decode graphs must contain kernel nodes only."""
from __future__ import annotations

import ctypes as C

import torch

from ..ops import _lib
from ..ops._lib import P, call


class NativeGraph:
    def __init__(self, body, pdl: bool = True, allow_non_kernel: bool = False):
        lib = _lib.load()
        lib.dgpp_graph_end_capture.restype = P
        lib.dgpp_graph_end_capture.argtypes = [P, C.c_int, C.c_int, P]
        self.stream = torch.cuda.Stream()
        self.stream.wait_stream(torch.cuda.current_stream())
        info = (C.c_int * 3)()
        with torch.cuda.stream(self.stream):
            call("dgpp_graph_begin_capture", self.stream.cuda_stream)
            try:
                body()
            finally:
                self.handle = lib.dgpp_graph_end_capture(self.stream.cuda_stream, int(pdl), int(allow_non_kernel),
                                                         C.cast(info, P))
        if not self.handle:
            raise RuntimeError("graph capture failed: " + lib.dgpp_last_error().decode())
        self.kernel_nodes, self.other_nodes, self.programmatic_edges = info[0], info[1], info[2]
        torch.cuda.current_stream().wait_stream(self.stream)

    def replay(self) -> None:
        call("dgpp_graph_launch", self.handle, torch.cuda.current_stream().cuda_stream)

    def __del__(self):
        try:
            if getattr(self, "handle", None):
                call("dgpp_graph_destroy", self.handle)
                self.handle = None
        except Exception:
            pass
