"""Native CUDA-graph executor (csrc/engine/graph_exec.cu): capture a launch sequence once, replay it with
programmatic-dependent-launch edges between the kernels.  Decode graphs must contain kernel nodes only."""
from __future__ import annotations

import ctypes as C

import torch

from ..ops import _lib
from ..ops._lib import P, call


def capture_with_pdl(body, pdl: bool = True):
    """Captures `body()` into a torch CUDA graph (private memory pool, so tensors created inside stay valid) and, before
    it is instantiated, rewrites the kernel -> kernel edges that end in a kernel of this library as programmatic
    dependent launches: those kernels wait for their predecessor themselves, so their prologue overlaps its tail.
    Edges into framework kernels stay plain.  Returns (graph, body's result, programmatic edge count)."""
    graph = torch.cuda.CUDAGraph(keep_graph=True) if pdl else torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        out = body()
    edges = 0
    if pdl:
        _lib.declare("dgpp_graph_pdl_rewrite", [P, P])
        info = (C.c_int * 3)()
        call("dgpp_graph_pdl_rewrite", graph.raw_cuda_graph(), C.cast(info, P))
        edges = info[2]
        graph.instantiate()
    return graph, out, edges


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

    def decode_loop(self, d_tokens: torch.Tensor, b: int, steps: int, inflight: int = 2, stop_ids=()):
        """Native step loop (csrc/engine/graph_exec.cu dgpp_decode_loop): `steps` replays with at most `inflight`
        outstanding, ids and the device status read back per step through a pinned mailbox, rows watched for stop ids.
        Returns (ids as a [delivered, b] int32 tensor on the host, per-row stop step or -1, steps launched)."""
        from ..ops._lib import I, ptr
        _lib.declare("dgpp_decode_loop", [P, P, I, I, I, P, I, P, P, P, P])
        out = torch.zeros(max(steps, 1), b, dtype=torch.int32)
        row_stop = torch.zeros(b, dtype=torch.int32)
        ran = (C.c_int * 2)()
        stops = (C.c_int32 * max(len(stop_ids), 1))(*stop_ids)
        call("dgpp_decode_loop", self.handle, ptr(d_tokens), b, steps, inflight, C.cast(stops, P), len(stop_ids),
             out.data_ptr(), row_stop.data_ptr(), C.cast(ran, P), torch.cuda.current_stream().cuda_stream)
        return out[:ran[0]], row_stop.tolist(), ran[1]

    def __del__(self):
        try:
            if getattr(self, "handle", None):
                call("dgpp_graph_destroy", self.handle)
                self.handle = None
        except Exception:
            pass
