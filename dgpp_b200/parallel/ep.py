"""Expert parallelism with token-sharded all-to-all dispatch / combine over NVLink peer memory.

Every rank routes ITS rows, stores each (token, k) pair's row into the receive area of the rank that owns the expert,
runs the grouped block-scaled expert GEMMs over what it received (sorted into 64-row tiles per local expert), stores the
result rows back into the sources' return areas, and folds its own rows' results in ascending k order.  All transfers
are plain peer stores from our kernels (`csrc/kernels/ep_moe.cu`) with bounded flag waits; NCCL only carries the IPC
handles at construction.  The result is bit-identical to the single-rank prefill path of `MoEBlock` whatever the number
of ranks: positions, tiles and fold order are functions of the routing result alone.
(reference counterparts: src/kernels/glm_moe.cu dispatch / combine, src/engine/tp_bus.hpp expert exchange.)
"""
from __future__ import annotations

import ctypes as C
from typing import Optional

import torch

from ..models.moe import MoEWeights
from ..ops import _lib
from ..ops import core as ops
from ..ops._lib import I, L, P, call, ptr, stream_ptr

BF = torch.bfloat16

_lib.declare("dgpp_ep_dispatch", [P, P, L, P, P, P, I, I, I, I, I, P])
_lib.declare("dgpp_ep_recv_plan", [P, P, P, P, I, I, I, I, P])
_lib.declare("dgpp_ep_gather", [P, P, P, P, I, I, I, I, P])
_lib.declare("dgpp_ep_return", [P, P, P, P, I, I, I, I, P])
_lib.declare("dgpp_ep_combine", [P, P, P, P, P, I, I, I, I, I, P])
_lib.declare("dgpp_comm_connect", [P, P])
_lib.declare("dgpp_comm_destroy", [P])


def open_comm(slot_bytes: int, device, group=None):
    """A symmetric peer-memory communicator with `slot_bytes` per (parity, source) slot.  Returns (handle, world, rank).
    Without an initialised process group the communicator is a single rank looping back to itself."""
    import torch.distributed as dist

    lib = _lib.load()
    lib.dgpp_comm_create.restype = P
    lib.dgpp_comm_create.argtypes = [I, I, L, P]
    multi = dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1
    world = dist.get_world_size(group) if multi else 1
    rank = dist.get_rank(group) if multi else 0
    handle = (C.c_ubyte * 64)()
    torch.cuda.set_device(device)
    comm = lib.dgpp_comm_create(world, rank, int(slot_bytes), C.cast(handle, P))
    if not comm:
        raise RuntimeError("comm_create: " + lib.dgpp_last_error().decode())
    blob = None
    if multi:
        mine = torch.tensor(list(bytes(handle)), dtype=torch.uint8, device=device)
        allh = [torch.empty_like(mine) for _ in range(world)]
        dist.all_gather(allh, mine, group=group)
        raw = b"".join(bytes(h.cpu().tolist()) for h in allh)
        blob = C.create_string_buffer(raw, len(raw))
        call("dgpp_comm_connect", comm, C.cast(blob, P))
        dist.barrier(group=group)
    return comm, world, rank, blob


class EpMoE:
    """One MoE block under expert parallelism.  `w` holds this rank's expert block (stacked) and, when the model has a
    shared expert, a copy of it (the shared expert runs on the rank's own rows)."""

    def __init__(self, w: MoEWeights, max_rows: int, device, group=None, act_terms: int = 3, comm=None, pool=None):
        """comm: a communicator from `open_comm` shared by the blocks of one model (their exchanges are sequential; the
        slot size must fit max_rows * top_k pairs); pool: a dict through which those blocks share their tile buffers."""
        c = w.cfg
        assert w.gu_q is not None, "call MoEWeights.stack() on the device first"
        self.w, self.c, self.dev, self.terms = w, c, device, act_terms
        self.max_rows, self.max_pairs = max_rows, max_rows * c.top_k
        lib = _lib.load()
        lib.dgpp_ep_slot_bytes.restype = L
        lib.dgpp_ep_slot_bytes.argtypes = [I, I]
        slot = lib.dgpp_ep_slot_bytes(c.hidden, self.max_pairs)
        self.slot_bytes = slot
        self.comm, self.world, self.rank, self._blob = comm if comm is not None else open_comm(slot, device, group)
        self.owns_comm = comm is None
        assert c.experts % self.world == 0, "experts must divide over the ranks"
        per = c.experts // self.world
        self.local = per
        assert (w.e_begin, w.e_end or c.experts) == (self.rank * per, (self.rank + 1) * per), "w is not this rank's expert block"
        cap = self.world * self.max_pairs
        self.bn = 64
        self.max_tiles = (cap + self.bn - 1) // self.bn + per
        i32 = dict(dtype=torch.int32, device=device)
        self.dest_pos, self.dest_cnt = torch.zeros(self.max_pairs, **i32), torch.zeros(8, **i32)
        self.recv_ids, self.recv_src = torch.full((cap,), -1, **i32), torch.full((cap,), -1, **i32)
        self.n_recv = torch.zeros(1 + 8, **i32)
        self.pair_row = torch.full((cap,), -1, **i32)
        self.tiles, self.n_tiles = torch.full((self.max_tiles,), -1, **i32), torch.zeros(1, **i32)
        rows = self.max_tiles * self.bn

        def shared(name, make):
            if pool is None:
                return make()
            key = (name, self.max_tiles, c.hidden, c.moe_ffn, act_terms)
            if key not in pool:
                pool[key] = make()
            return pool[key]

        self.xs = shared("xs", lambda: torch.zeros(rows, c.hidden, dtype=BF, device=device))
        self.h = shared("h", lambda: torch.zeros(self.max_tiles, self.bn, 2 * c.moe_ffn, dtype=BF, device=device))
        self.y = shared("y", lambda: torch.zeros(self.max_tiles, self.bn, c.hidden, dtype=BF, device=device))
        self.qa_x = shared("qa_x", lambda: ops.QuantAct(rows, c.hidden, act_terms, self.bn, device))
        self.qa_mid = shared("qa_mid", lambda: ops.QuantAct(rows, c.moe_ffn, act_terms, self.bn, device))

    def forward(self, xn: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """xn: this rank's rows [T, H] bf16 (1 <= T <= max_rows; every rank calls with its own T).  Returns [T, H]."""
        c, w = self.c, self.w
        T = xn.shape[0]
        assert 1 <= T <= self.max_rows and xn.dtype == BF
        k, H, E, mp = c.top_k, c.hidden, c.experts, self.max_pairs
        ids, wts = ops.moe_route(xn, w.gate, w.bias, k, c.n_group, c.topk_group, c.router == "softmax", c.norm_topk_prob,
                                 c.routed_scaling)
        st = stream_ptr()
        call("dgpp_ep_dispatch", self.comm, ptr(xn), xn.stride(0), ptr(ids), ptr(self.dest_pos), ptr(self.dest_cnt), T, k, H,
             E, mp, st)
        call("dgpp_ep_recv_plan", self.comm, ptr(self.recv_ids), ptr(self.recv_src), ptr(self.n_recv), k, H, E, mp, st)
        cap = self.world * mp
        ops.moe_segment_sort(self.recv_ids.view(cap, 1), self.bn, self.max_tiles, 0, self.local, self.pair_row, self.tiles,
                             self.n_tiles)
        call("dgpp_ep_gather", self.comm, ptr(self.recv_src), ptr(self.pair_row), ptr(self.xs), k, H, E, mp, st)
        rows = self.max_tiles * self.bn
        xa = ops.act_quant_nvfp4(self.xs, self.terms, out=self.qa_x, group_list=self.tiles, group_rows=self.bn)
        ops.gemm_fp4_grouped(xa, w.gu_q, w.gu_sf, w.gu_alpha, self.h, self.bn, 2 * c.moe_ffn, H, self.local, self.tiles,
                             group_b=True)
        xm = ops.act_quant_nvfp4(self.h.view(rows, 2 * c.moe_ffn), self.terms, out=self.qa_mid, mode="swiglu",
                                 limit=c.swiglu_limit, alpha=c.swiglu_alpha, group_list=self.tiles, group_rows=self.bn)
        ops.gemm_fp4_grouped(xm, w.down_q, w.down_sf, w.down_alpha, self.y, self.bn, H, c.moe_ffn, self.local, self.tiles,
                             group_b=True)
        call("dgpp_ep_return", self.comm, ptr(self.recv_src), ptr(self.pair_row), ptr(self.y), k, H, E, mp, st)
        sh = None
        if w.shared_gu is not None:
            sh = ops.linear(ops.swiglu(ops.linear(xn, w.shared_gu_k or w.shared_gu), limit=c.swiglu_limit, alpha=c.swiglu_alpha),
                            w.shared_down_k or w.shared_down)
        if out is None:
            out = torch.empty(T, H, dtype=BF, device=xn.device)
        call("dgpp_ep_combine", self.comm, ptr(ids), ptr(wts), ptr(sh), ptr(out), T, k, H, E, mp, st)
        return out

    def nvlink_bytes_per_row(self) -> float:
        """Bytes one row moves over NVLink per block: k pair rows out and k result rows back, except the share whose expert
        is local (1 / world on average) -- against 2 (world - 1) / world rows of H values for a ring all-reduce."""
        c = self.c
        return 2.0 * c.top_k * c.hidden * 2 * (self.world - 1) / self.world

    def close(self) -> None:
        if self.comm and self.owns_comm:
            call("dgpp_comm_destroy", self.comm)
            self.comm = None
