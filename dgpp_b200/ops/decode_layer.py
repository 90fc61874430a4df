"""ctypes front end of the persistent decode-layer kernel (``csrc/kernels/decode_layer.cu``).

A `LayerLaunch` is one launch: an ordered list of phases over static buffers.  It is built once (all pointers are
those of preallocated tensors) and replayed by `launch()`; inside a captured decode graph it is one kernel node.
"""
from __future__ import annotations

import ctypes as C
from typing import Optional

import torch

from . import _lib
from ._lib import ptr, stream_ptr

PH_ROWA, PH_GEMM, PH_UNITQ, PH_ROPE, PH_ROWC = 1, 2, 3, 4, 5
MAX_PHASE, MAX_GEMM, MAX_ACT, MAX_ROWQ = 16, 4, 3, 3
MAX_ROWS = 16


class _Act(C.Structure):
    _fields_ = [("q", C.c_void_p), ("sf", C.c_void_p), ("g", C.c_void_p), ("K", C.c_int), ("pad", C.c_int)]


class _Gemm(C.Structure):
    _fields_ = [("wq", C.c_void_p), ("wsf", C.c_void_p), ("alpha", C.c_float), ("N", C.c_int), ("K", C.c_int),
                ("pair", C.c_int), ("act", C.c_int), ("splits", C.c_int)]


class _Rowq(C.Structure):
    _fields_ = [("mode", C.c_int), ("src_gemm", C.c_int), ("out_act", C.c_int), ("tp_fold", C.c_int),
                ("inp", C.c_void_p), ("in_stride", C.c_int64), ("norm_w", C.c_void_p), ("x_out", C.c_void_p)]


class _Args(C.Structure):
    _fields_ = [
        ("rows", C.c_int), ("nphase", C.c_int),
        ("ph_type", C.c_int * MAX_PHASE), ("ph_idx", C.c_int * MAX_PHASE),
        ("gemm", _Gemm * MAX_GEMM), ("act", _Act * MAX_ACT), ("rowq", _Rowq * MAX_ROWQ),
        ("x", C.c_void_p), ("H", C.c_int), ("eps", C.c_float), ("limit", C.c_float), ("one_plus_w", C.c_int),
        ("ws", C.c_void_p), ("ws_floats", C.c_int64), ("hbuf", C.c_void_p), ("amax_part", C.c_void_p),
        ("stats", C.c_void_p), ("unitq_act", C.c_int), ("inter", C.c_int),
        ("part_ml", C.c_void_p), ("part_acc", C.c_void_p), ("att_splits", C.c_int), ("hq", C.c_int), ("d", C.c_int),
        ("rope_gemm", C.c_int), ("hkv", C.c_int),
        ("qkv", C.c_void_p), ("positions", C.c_void_p), ("row_req", C.c_void_p), ("block_table", C.c_void_p),
        ("inv_freq", C.c_void_p), ("q_norm_w", C.c_void_p), ("k_norm_w", C.c_void_p),
        ("k_cache", C.c_void_p), ("v_cache", C.c_void_p), ("k_scale", C.c_void_p), ("v_scale", C.c_void_p),
        ("rot_dim", C.c_int), ("page", C.c_int), ("max_blocks", C.c_int), ("kv_fp8", C.c_int),
        ("mscale", C.c_float), ("grid", C.c_int), ("comm", C.c_void_p),
    ]


_declared = False


def _declare():
    global _declared
    if not _declared:
        _lib.declare("dgpp_decode_layer", [C.c_void_p, C.c_void_p])
        _lib.declare("dgpp_decode_layer_reset", [C.c_void_p])
        _declared = True


def reset() -> None:
    """Zero the grid-barrier words of the current device (needed after a launch that reported a failure)."""
    _declare()
    _lib.call("dgpp_decode_layer_reset", stream_ptr())


def sm_count() -> int:
    lib = _lib.load()
    lib.dgpp_decode_layer_grid.restype = C.c_int
    lib.dgpp_decode_layer_grid.argtypes = []
    return int(lib.dgpp_decode_layer_grid())


def stage_tiled(w) -> torch.Tensor:
    """The packed e2m1 payload [N, K / 2] of `w` re-ordered as [N / 128][K / 256][128 rows][128 bytes]: every
    (128 rows x 256 K) pipeline stage becomes 16 KB of contiguous memory.  A byte permutation of the checkpoint
    payload, made once and cached on the matrix."""
    t = getattr(w, "_stage_tiled", None)
    if t is None:
        n, kb = w.payload.shape
        t = w.payload.view(n // 128, 128, kb // 128, 128).permute(0, 2, 1, 3).contiguous()
        w._stage_tiled = t
    return t


class LayerLaunch:
    """Builder of one launch: an ordered list of phases over static buffers.  Activation buffers are
    `ops.core.QuantAct` objects with bn = 16 and 3 terms; weights are `QuantLinear` (nvfp4).  Tensors handed in must
    outlive the object (it keeps references)."""

    def __init__(self, rows: int, x: Optional[torch.Tensor], hidden: int, eps: float, ws: torch.Tensor,
                 stats: torch.Tensor, one_plus_w: bool = False, limit: float = 0.0, comm=None, grid: int = 0):
        assert 1 <= rows <= MAX_ROWS
        _declare()
        self.a = _Args()
        assert stats.numel() >= 256 and stats.dtype == torch.float32
        self.keep = [x, ws, stats]
        a = self.a
        a.rows, a.nphase = rows, 0
        a.x, a.H, a.eps, a.limit, a.one_plus_w = ptr(x), hidden, float(eps), float(limit), int(one_plus_w)
        a.ws, a.ws_floats, a.stats = ptr(ws), ws.numel(), ptr(stats)
        a.unitq_act, a.rope_gemm = -1, -1
        a.grid = grid
        a.comm = comm
        for i in range(MAX_ROWQ):
            a.rowq[i].src_gemm = -1
            a.rowq[i].out_act = -1

    def _phase(self, t: int, idx: int):
        a = self.a
        assert a.nphase < MAX_PHASE
        a.ph_type[a.nphase], a.ph_idx[a.nphase] = t, idx
        a.nphase += 1

    def set_act(self, idx: int, qa) -> None:
        assert qa.bn == 16 and qa.terms == 3 and qa.rows_pad == 16, "decode-layer kernel takes 16-row, 3-term buffers"
        s = self.a.act[idx]
        s.q, s.sf, s.g, s.K = ptr(qa.q), ptr(qa.sf), ptr(qa.g), qa.k
        self.keep.append(qa)

    def set_gemm(self, idx: int, w, act: int, pair: bool = False, splits: int = 0) -> None:
        assert w.fmt == "nvfp4" and w.n % 128 == 0 and w.k % 256 == 0
        g = self.a.gemm[idx]
        sf, wt = w.tiled_scales(), stage_tiled(w)
        g.wq, g.wsf, g.alpha, g.N, g.K = ptr(wt), ptr(sf), float(w.alpha), w.n, w.k
        g.pair, g.act, g.splits = int(pair), act, splits
        self.keep += [w, sf, wt]

    def rowq(self, idx: int, mode: int, out_act: int = -1, src_gemm: int = -1, tp_fold: bool = False, inp=None,
             norm_w=None, x_out=None) -> None:
        """Row phase `idx` (two steps: produce + statistics, then finish + quantise)."""
        r = self.a.rowq[idx]
        r.mode, r.src_gemm, r.out_act, r.tp_fold = mode, src_gemm, out_act, int(tp_fold)
        r.inp, r.in_stride = ptr(inp), (inp.stride(0) if inp is not None else 0)
        r.norm_w, r.x_out = ptr(norm_w), ptr(x_out)
        self.keep += [inp, norm_w, x_out]
        self._phase(PH_ROWA, idx)
        self._phase(PH_ROWC, idx)

    def gemm(self, idx: int) -> None:
        self._phase(PH_GEMM, idx)

    def set_attention(self, part_ml, part_acc, splits: int, hq: int, d: int) -> None:
        a = self.a
        a.part_ml, a.part_acc, a.att_splits, a.hq, a.d = ptr(part_ml), ptr(part_acc), splits, hq, d
        self.keep += [part_ml, part_acc]

    def set_swiglu(self, hbuf: torch.Tensor, amax_part: torch.Tensor, inter: int, out_act: int) -> None:
        a = self.a
        assert amax_part.numel() >= (inter // 128) * 16 and hbuf.numel() >= a.rows * inter
        a.hbuf, a.amax_part, a.inter, a.unitq_act = ptr(hbuf), ptr(amax_part), inter, out_act
        self.keep += [hbuf, amax_part]

    def unitq(self) -> None:
        self._phase(PH_UNITQ, 0)

    def rope(self, gemm_idx: int, qkv, positions, row_req, block_table, inv_freq, cache, hq: int, hkv: int, d: int,
             rot_dim: int, mscale: float, q_norm_w=None, k_norm_w=None) -> None:
        a = self.a
        a.rope_gemm, a.hq, a.hkv, a.d = gemm_idx, hq, hkv, d
        a.qkv, a.positions, a.row_req, a.block_table = ptr(qkv), ptr(positions), ptr(row_req), ptr(block_table)
        a.inv_freq, a.q_norm_w, a.k_norm_w = ptr(inv_freq), ptr(q_norm_w), ptr(k_norm_w)
        a.k_cache, a.v_cache = ptr(cache.k), ptr(cache.v)
        a.k_scale, a.v_scale = ptr(cache.k_scale), ptr(cache.v_scale)
        a.rot_dim, a.page, a.max_blocks, a.kv_fp8 = rot_dim, cache.page, block_table.shape[1], int(cache.fp8)
        a.mscale = float(mscale)
        self.keep += [qkv, positions, row_req, block_table, inv_freq, q_norm_w, k_norm_w, cache]
        self._phase(PH_ROPE, 0)

    def launch(self) -> None:
        _lib.call("dgpp_decode_layer", C.addressof(self.a), stream_ptr())
