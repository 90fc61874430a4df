"""Tensor-parallel reductions done by our own kernels over NVLink peer memory (CUDA IPC symmetric regions).

``PeerReducer`` has the interface of ``NcclReducer`` (``all_reduce``, ``merge_picks``) but every call is one
kernel launch of ``csrc/kernels/comm.cu``: push to the peers' regions, flag, bounded wait, fixed-order fold.
Handles are exchanged once through ``torch.distributed`` (any backend) at construction.
"""
from __future__ import annotations

import ctypes as C

import torch
import torch.distributed as dist

from ..ops import _lib
from ..ops._lib import F, I, L, P, call, ptr, stream_ptr

_lib.declare("dgpp_comm_connect", [P, P])
_lib.declare("dgpp_comm_destroy", [P])
_lib.declare("dgpp_comm_all_reduce", [P, P, P, L, I, P])
_lib.declare("dgpp_comm_pick_merge", [P, P, P, I, P])
_lib.declare("dgpp_comm_rs_ag", [P, P, I, I, I, P])
_lib.declare("dgpp_comm_rs_norm_push", [P, P, P, F, I, I, I, I, P])


class PeerReducer:
    launches_per_all_reduce = 1

    def __init__(self, hidden: int, max_rows: int, device, group=None, ctas: int = 16):
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.ctas = ctas
        self.max_values = hidden * max_rows
        slot = (self.max_values * 2 + 255) // 256 * 256
        lib = _lib.load()
        lib.dgpp_comm_create.restype = P
        lib.dgpp_comm_create.argtypes = [I, I, L, P]
        handle = (C.c_ubyte * 64)()
        torch.cuda.set_device(device)
        self.comm = lib.dgpp_comm_create(self.world, self.rank, slot, C.cast(handle, P))
        if not self.comm:
            raise RuntimeError("comm_create: " + lib.dgpp_last_error().decode())
        mine = torch.tensor(list(bytes(handle)), dtype=torch.uint8, device=device)
        allh = [torch.empty_like(mine) for _ in range(self.world)]
        dist.all_gather(allh, mine, group=group)
        blob = b"".join(bytes(h.cpu().tolist()) for h in allh)
        self._blob = C.create_string_buffer(blob, len(blob))
        call("dgpp_comm_connect", self.comm, C.cast(self._blob, P))
        dist.barrier(group=group)

    def all_reduce(self, t: torch.Tensor, resid: torch.Tensor | None = None) -> torch.Tensor:
        n = t.numel()
        assert t.is_contiguous() and t.dtype == torch.bfloat16
        if n > self.max_values:
            # prefill-sized tensors: reduce in slot-sized pieces
            flat = t.view(-1)
            step = self.max_values
            for o in range(0, n, step):
                m = min(step, n - o)
                call("dgpp_comm_all_reduce", self.comm, ptr(flat[o:o + m]),
                     None if resid is None else ptr(resid.view(-1)[o:o + m]), m, 64, stream_ptr())
            return t
        ctas = self.ctas if n <= 64 * 8192 else 64
        call("dgpp_comm_all_reduce", self.comm, ptr(t), ptr(resid), n, ctas, stream_ptr())
        return t

    def rs_ag(self, x: torch.Tensor, tile_rows: int) -> torch.Tensor:
        """Second half of the fused GEMM -> reduce-scatter -> all-gather: x [T, H] += the sum over ranks of the
        partial tiles that ``ops.gemm_tc_push`` delivered (fixed-order fold at the owner, then broadcast)."""
        assert x.is_contiguous() and x.dtype == torch.bfloat16
        call("dgpp_comm_rs_ag", self.comm, ptr(x), x.shape[0], x.shape[1], tile_rows, stream_ptr())
        return x

    def rs_norm_push(self, x: torch.Tensor, norm_w: torch.Tensor, eps: float, tile_rows: int, one_plus_w: bool = False) -> None:
        """Sequence-parallel boundary after ``ops.gemm_tc_push``: this rank folds the partial tiles of ITS token tiles
        into x (the other rows of x are left as they are: no rank needs them), normalises those rows and stores the
        normed rows into every rank's region; the next projection reads them with ``ops.gemm_tc_ag``."""
        assert x.is_contiguous() and x.dtype == torch.bfloat16
        call("dgpp_comm_rs_norm_push", self.comm, ptr(x), ptr(norm_w), float(eps), int(one_plus_w), x.shape[0], x.shape[1],
             tile_rows, stream_ptr())

    def can_rs(self, rows: int, hidden: int, tile_rows: int) -> bool:
        return (rows * hidden <= self.max_values and hidden % 128 == 0 and (rows + tile_rows - 1) // tile_rows <= 64)

    def merge_picks(self, ids: torch.Tensor, vals: torch.Tensor) -> None:
        call("dgpp_comm_pick_merge", self.comm, ptr(ids), ptr(vals), ids.numel(), stream_ptr())

    def close(self) -> None:
        if self.comm:
            call("dgpp_comm_destroy", self.comm)
            self.comm = None
