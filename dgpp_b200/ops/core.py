"""Python entry points of the sm_100a kernels (thin: pointer marshalling and shape checks only)."""
from __future__ import annotations

import math
import os
from typing import Optional

import torch

from ..quant.formats import QuantLinear
from . import _lib
from ._lib import F, I, L, P, call, ptr, stream_ptr

_FMT_GEMV = {"nvfp4": 0, "mxfp4": 1, "bf16": 2}
_FMT_GEMM = {"bf16": 0, "nvfp4": 1, "fp8": 2, "mxfp4": 3, "mxfp8": 4, "int8": 5, "int4": 6, "bf12": 7}

# The converted-weight operand is always bf16: tcgen05 kind::f16 takes A and B of one 16-bit type.
A_F16_DEFAULT = 0


def _chk(t: torch.Tensor, dtype, name: str):
    if t.dtype != dtype:
        raise TypeError(f"{name}: expected {dtype}, got {t.dtype}")
    if not t.is_cuda:
        raise RuntimeError(f"{name}: CUDA tensor required")


def embed_gather(ids: torch.Tensor, table: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    _chk(ids, torch.int32, "ids")
    _chk(table, torch.bfloat16, "table")
    rows, (vocab, hidden) = ids.numel(), table.shape
    if out is None:
        out = torch.empty(rows, hidden, dtype=torch.bfloat16, device=table.device)
    call("dgpp_embed_gather", ptr(ids), ptr(table), ptr(out), rows, hidden, vocab, stream_ptr())
    return out


def add(a: torch.Tensor, b: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """out = bf16(a + b), element by element (contiguous bf16 tensors of one shape; out may be a)."""
    _chk(a, torch.bfloat16, "a")
    _chk(b, torch.bfloat16, "b")
    if out is None:
        out = torch.empty_like(a)
    call("dgpp_add_bf16", ptr(a), ptr(b), ptr(out), a.numel(), stream_ptr())
    return out


def rmsnorm(x: torch.Tensor, w: torch.Tensor, eps: float = 1e-6, delta: Optional[torch.Tensor] = None,
            resid_out: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None,
            one_plus_w: bool = False):
    """out = rmsnorm(x [+ delta]).  With `delta` the sum is written to `resid_out` (default: x, in place)."""
    _chk(x, torch.bfloat16, "x")
    rows, hidden = x.shape
    if out is None:
        out = torch.empty_like(x)
    if delta is not None and resid_out is None:
        resid_out = x
    call("dgpp_rmsnorm", ptr(x), ptr(delta), ptr(w), ptr(resid_out), ptr(out), rows, hidden, float(eps),
         int(one_plus_w), stream_ptr())
    return out


def swiglu(gate_up: torch.Tensor, out: Optional[torch.Tensor] = None, limit: float = 0.0, alpha: float = 0.0) -> torch.Tensor:
    _chk(gate_up, torch.bfloat16, "gate_up")
    rows, two_i = gate_up.shape
    inter = two_i // 2
    if out is None:
        out = torch.empty(rows, inter, dtype=torch.bfloat16, device=gate_up.device)
    call("dgpp_swiglu", ptr(gate_up), ptr(out), rows, inter, float(limit), float(alpha), stream_ptr())
    return out


def argmax(logits: torch.Tensor, id_base: int = 0, out_id: Optional[torch.Tensor] = None,
           out_val: Optional[torch.Tensor] = None):
    rows, vocab = logits.shape
    dt = {torch.bfloat16: 0, torch.float32: 1}[logits.dtype]
    if out_id is None:
        out_id = torch.empty(rows, dtype=torch.int32, device=logits.device)
    if out_val is None:
        out_val = torch.empty(rows, dtype=torch.float32, device=logits.device)
    call("dgpp_argmax", ptr(logits), dt, logits.stride(0), rows, vocab, id_base, ptr(out_id), ptr(out_val),
         stream_ptr())
    return out_id, out_val


def gemv(x: torch.Tensor, w: QuantLinear, out: Optional[torch.Tensor] = None,
         out32: Optional[torch.Tensor] = None) -> torch.Tensor:
    """CUDA-core weight-streaming GEMV, rows <= 4."""
    _chk(x, torch.bfloat16, "x")
    rows, k = x.shape
    assert k == w.k and w.fmt in _FMT_GEMV
    if out is None and out32 is None:
        out = torch.empty(rows, w.n, dtype=torch.bfloat16, device=x.device)
    ys = (out if out is not None else out32).stride(0)
    call("dgpp_gemv_quant", _FMT_GEMV[w.fmt], ptr(x), ptr(w.payload), ptr(w.scale), float(w.alpha), ptr(out),
         ptr(out32), rows, w.n, k, x.stride(0), ys, stream_ptr())
    return out if out is not None else out32


class GemmWorkspace:
    """Split-K scratch for ``gemm_tc``: fp32 partials and per-tile arrival counters (zero at rest)."""

    def __init__(self, device, max_partial_floats: int = 1 << 24, max_tiles: int = 1 << 16):
        self.partials = torch.empty(max_partial_floats, dtype=torch.float32, device=device)
        self.counters = torch.zeros(max_tiles, dtype=torch.int32, device=device)


_WS: dict = {}


def default_workspace(device) -> GemmWorkspace:
    key = str(device)
    if key not in _WS:
        _WS[key] = GemmWorkspace(device)
    return _WS[key]


def pick_bn(rows: int) -> int:
    for bn in (16, 32, 64, 128):
        if rows <= bn:
            return bn
    return 256


def pick_splits(rows: int, n: int, k: int, bn: int, sms: int = 148) -> int:
    """Split K until the grid covers the SMs (weight-streaming regime only)."""
    tiles = math.ceil(n / 128) * math.ceil(rows / bn)
    if tiles >= sms or rows > 128:
        return 1
    kb = k // 64
    want = max(1, sms // tiles)
    return max(1, min(want, kb // 8))


# 4-bit weights at prefill sizes can run on CTA pairs (`gemm_tc_pair.cu`: 256 weight rows x 256 tokens per pair, each
# SM loading half of the activation tile); results are bit-identical to the single-CTA kernel.  Off by default: it
# measured slower (537 against 596-662 TFLOP/s at 2048 x 34816 x 5120).
PAIR_GEMM = False
PAIR_GEMM_MIN_ROWS = 512

_lib.declare("dgpp_gemm_tc_pair", [I, P, L, P, P, F, P, P, I, I, I, I, P])


def gemm_tc_pair(x: torch.Tensor, w: QuantLinear, out: Optional[torch.Tensor] = None,
                 resid: Optional[torch.Tensor] = None) -> torch.Tensor:
    """The W4A16 linear on CTA pairs (NVFP4 / MXFP4 weights, N a multiple of 256)."""
    _chk(x, torch.bfloat16, "x")
    rows, k = x.shape
    assert k == w.k and w.fmt in ("nvfp4", "mxfp4") and w.n % 256 == 0 and k % 256 == 0
    if out is None:
        out = torch.empty(rows, w.n, dtype=torch.bfloat16, device=x.device)
    call("dgpp_gemm_tc_pair", _FMT_GEMM[w.fmt], ptr(x), x.stride(0), ptr(w.payload), ptr(w.scale), float(w.alpha), ptr(out),
         ptr(resid), out.stride(0), rows, w.n, k, stream_ptr())
    return out


def gemm_tc(x: torch.Tensor, w: QuantLinear, out: Optional[torch.Tensor] = None,
            out32: Optional[torch.Tensor] = None, resid: Optional[torch.Tensor] = None,
            bn: Optional[int] = None, splits: Optional[int] = None, a_f16: Optional[int] = None,
            ws: Optional[GemmWorkspace] = None) -> torch.Tensor:
    """tcgen05 linear: out[T, N] = alpha * x[T, K] @ dequant(w)[N, K]^T (+ resid)."""
    _chk(x, torch.bfloat16, "x")
    rows, k = x.shape
    assert k == w.k, (k, w.k)
    assert w.fmt in _FMT_GEMM, w.fmt
    if (PAIR_GEMM and out32 is None and bn is None and splits in (None, 1) and rows >= PAIR_GEMM_MIN_ROWS
            and w.fmt in ("nvfp4", "mxfp4") and w.n % 256 == 0 and k % 256 == 0):
        return gemm_tc_pair(x, w, out=out, resid=resid)
    if out is None and out32 is None:
        out = torch.empty(rows, w.n, dtype=torch.bfloat16, device=x.device)
    ldc = (out if out is not None else out32).stride(0)
    if bn is None:
        bn = pick_bn(rows)
    if splits is None:
        splits = pick_splits(rows, w.n, k, bn)
    if a_f16 is None:
        a_f16 = A_F16_DEFAULT if w.fmt == "nvfp4" else 0
    wsp = cnt = None
    if splits > 1:
        ws = ws or default_workspace(x.device)
        need = splits * rows * w.n
        tiles = math.ceil(w.n / 128) * math.ceil(rows / bn)
        if need > ws.partials.numel() or tiles > ws.counters.numel():
            splits = 1
        else:
            wsp, cnt = ws.partials, ws.counters
    call("dgpp_gemm_tc", _FMT_GEMM[w.fmt], int(a_f16), bn, ptr(x), x.stride(0), ptr(w.payload), ptr(w.scale),
         float(w.alpha), ptr(out), ptr(out32), ptr(resid), ldc, rows, w.n, k, splits, ptr(wsp), ptr(cnt),
         stream_ptr())
    return out if out is not None else out32


def gemm_tc_push(x: torch.Tensor, w: QuantLinear, push_comm, bn: Optional[int] = None) -> int:
    """The same linear with the reduce-scatter epilogue: every finished bf16 tile is stored into the symmetric
    region of the rank that owns the tile's tokens (native peer communicator `push_comm`).  Returns the token tile
    size, which the matching ``PeerReducer.rs_ag`` call needs."""
    _chk(x, torch.bfloat16, "x")
    rows, k = x.shape
    assert k == w.k and w.fmt in _FMT_GEMM
    bn = bn or pick_bn(rows)
    call("dgpp_gemm_tc_push", _FMT_GEMM[w.fmt], 0, bn, ptr(x), x.stride(0), ptr(w.payload), ptr(w.scale), float(w.alpha),
         rows, w.n, k, push_comm, stream_ptr())
    return bn


def gemm_tc_ag(w: QuantLinear, ag_comm, rows: int, out: Optional[torch.Tensor] = None, bn: Optional[int] = None,
               splits: int = 1) -> torch.Tensor:
    """The linear whose activations are the normed rows of the sequence-parallel all-gather: every rank's
    ``PeerReducer.rs_norm_push`` (same token tile `bn`) stored them into this rank's symmetric region; a token tile of
    another rank is waited for inside the kernel (its TMA producer warp), this rank's own tiles run first."""
    assert w.fmt in _FMT_GEMM
    bn = bn or pick_bn(rows)
    if out is None:
        out = torch.empty(rows, w.n, dtype=torch.bfloat16, device=w.payload.device)
    a_f16 = A_F16_DEFAULT if w.fmt == "nvfp4" else 0
    call("dgpp_gemm_tc_ag", _FMT_GEMM[w.fmt], int(a_f16), bn, ag_comm, ptr(w.payload), ptr(w.scale), float(w.alpha), ptr(out),
         None, out.stride(0), rows, w.n, w.k, 1, None, None, stream_ptr())
    return out


class QuantAct:
    """Activations quantised to R residual NVFP4 terms: x ~= g[t] * sum_r dequant(term r).
    Rows of `q` are ordered [token tile][term][token in tile] (the B operand of one MMA is a token tile with its
    terms stacked); `sf` holds the e4m3 block scales in tcgen05.cp atom order per token tile; g: [rows_pad].
    With more than one term the whole batch must fit one token tile (decode)."""

    def __init__(self, rows_pad: int, k: int, terms: int, bn: int, device):
        assert rows_pad % bn == 0 and terms * bn <= 256
        atoms = 2 if terms * bn > 128 else 1
        self.q = torch.zeros(rows_pad * terms, k // 2, dtype=torch.uint8, device=device)
        self.sf = torch.zeros((rows_pad // bn) * (k // 256) * 4 * atoms * 512, dtype=torch.uint8, device=device)
        self.g = torch.ones(rows_pad, dtype=torch.float32, device=device)
        self.rows, self.k, self.terms, self.bn, self.rows_pad = 0, k, terms, bn, rows_pad

    def dequant(self) -> torch.Tensor:
        from ..quant.formats import e2m1_decode, unpack_nibbles, untile_scales
        tiles, R, bn, k = self.rows_pad // self.bn, self.terms, self.bn, self.k
        v = e2m1_decode(unpack_nibbles(self.q)).view(tiles, R, bn, k // 16, 16)
        sf = untile_scales(self.sf, tiles * R * bn, k // 16, R * bn).view(tiles, R, bn, k // 16)
        x = (v * sf.view(torch.float8_e4m3fn).float().unsqueeze(-1)).sum(1).reshape(tiles * bn, k)
        return x[:self.rows] * self.g[:self.rows].unsqueeze(-1)


def act_quant_nvfp4(x: torch.Tensor, terms: int = 3, out: Optional[QuantAct] = None, bn: Optional[int] = None,
                    mode: str = "plain", delta=None, norm_w=None, resid_out=None, x_out=None, eps: float = 1e-6,
                    limit: float = 0.0, one_plus_w: bool = False, fold_comm=None, group_list=None,
                    group_rows: int = 0, alpha: float = 0.0) -> QuantAct:
    """Quantise rows to residual NVFP4 terms, optionally fused with the producing operator:
    mode "plain": x [T, K];  "swiglu": x = [gate | up] [T, 2K];  "rmsnorm": x = residual [T, K] (+ delta), norm_w.
    fold_comm (rmsnorm mode): native peer-communicator handle; the delta is then the fixed-order fold of the tiles
    the tensor-parallel GEMMs pushed into this rank's symmetric region (see gemm_fp4 push_comm)."""
    _chk(x, torch.bfloat16, "x")
    rows = x.shape[0]
    k = x.shape[1] // 2 if mode == "swiglu" else x.shape[1]
    if out is None:
        bn = bn or min(pick_bn(rows), 64 if terms > 1 else 256)
        out = QuantAct((rows + bn - 1) // bn * bn, k, terms, bn, x.device)
    out.rows = rows
    assert rows <= out.rows_pad and out.k == k
    m = {"plain": 0, "swiglu": 1, "rmsnorm": 2}[mode]
    if m == 2 and (delta is not None or fold_comm) and resid_out is None:
        resid_out = x
    # a cluster per row spreads a decode batch over the SMs; bulk rows (prefill tiles) take one CTA per row instead.
    # Modes 0 / 1 reduce with max only, so their result does not depend on the split; the norm's sum of squares does,
    # and keeps the decode split at every row count.
    order = (1, 2, 4, 8) if (rows > 64 and m != 2) else (8, 4, 2, 1)
    cl = next((c for c in order if k % c == 0 and (k // c) % 16 == 0 and (k // c) * 2 <= 48 * 1024), 0)
    if cl:
        call("dgpp_act_quant_nvfp4_cluster", m, ptr(x), x.stride(0), ptr(delta), ptr(norm_w), ptr(resid_out),
             ptr(x_out), ptr(out.q), ptr(out.sf), ptr(out.g), rows, out.rows_pad, k, out.terms, out.bn, cl,
             float(eps), float(limit), float(alpha), int(one_plus_w), fold_comm, ptr(group_list), group_rows,
             stream_ptr())
    else:
        assert not fold_comm and group_list is None, "the all-reduce fold needs the cluster quantiser"
        call("dgpp_act_quant_nvfp4", m, ptr(x), x.stride(0), ptr(delta), ptr(norm_w), ptr(resid_out), ptr(x_out),
             ptr(out.q), ptr(out.sf), ptr(out.g), rows, out.rows_pad, k, out.terms, out.bn, float(eps),
             float(limit), float(alpha), int(one_plus_w), stream_ptr())
    return out


class DecodeQuant:
    """Decode-width passes (<= 16 rows) run their NVFP4 linears on the block-scaled tensor path: the producing norm /
    activation kernel writes the rows as three residual NVFP4 terms (near-bf16 together), one GEMM streams the packed
    weights as stored.  One QuantAct per input width, reused by every layer (a layer's passes are sequential)."""
    ROWS, TERMS = 16, 3

    def __init__(self, device):
        self.dev, self.bufs = device, {}

    def usable(self, rows: int, *ws) -> bool:
        return (rows <= self.ROWS and torch.device(self.dev).type == "cuda"
                and all(w is not None and w.fmt == "nvfp4" and w.k % 256 == 0 for w in ws))

    def buf(self, k: int, tag: str = "") -> QuantAct:
        key = (k, tag)
        if key not in self.bufs:
            self.bufs[key] = QuantAct(self.ROWS, k, self.TERMS, self.ROWS, self.dev)
        return self.bufs[key]

    def plain(self, x: torch.Tensor, tag: str = "") -> QuantAct:
        return act_quant_nvfp4(x, self.TERMS, out=self.buf(x.shape[1], tag))

    def norm(self, x, w, eps, delta=None, x_out=None, tag: str = "") -> QuantAct:
        """rmsnorm(x [+ delta]) -> terms (+ the bf16 normed rows in x_out); with a delta the sum is written back to x."""
        return act_quant_nvfp4(x, self.TERMS, out=self.buf(x.shape[1], tag), mode="rmsnorm", delta=delta, norm_w=w,
                                   x_out=x_out, eps=eps)

    def swiglu(self, gate_up: torch.Tensor, limit: float = 0.0, tag: str = "") -> QuantAct:
        return act_quant_nvfp4(gate_up, self.TERMS, out=self.buf(gate_up.shape[1] // 2, tag), mode="swiglu", limit=limit)


def attn_combine_quant(scratch, rows: int, splits: int, hq: int, d: int, out: QuantAct, x_out=None) -> QuantAct:
    """Fold the split-KV partials of a decode-attention pass (attn_decode_tc(..., partials_only=True)) and quantise
    the attention output rows [rows, hq * d] to residual NVFP4 terms in one launch; same arithmetic as the stand-alone
    combine followed by the plain quantiser.  x_out (optional, bf16 [rows, hq * d]) also receives the rows."""
    ml, acc = scratch
    k = hq * d
    assert out.k == k and rows <= out.rows_pad and k % 256 == 0
    out.rows = rows
    cl = next(c for c in (8, 4, 2, 1) if k % c == 0 and (k // c) % 16 == 0 and (k // c) * 2 <= 48 * 1024)
    call("dgpp_attn_combine_quant", ptr(ml), ptr(acc), splits, hq, d, ptr(x_out), ptr(out.q), ptr(out.sf), ptr(out.g),
         rows, out.rows_pad, out.terms, out.bn, cl, stream_ptr())
    return out


def gemm_fp4(xa: QuantAct, w: QuantLinear, out: Optional[torch.Tensor] = None,
             out32: Optional[torch.Tensor] = None, resid: Optional[torch.Tensor] = None,
             splits: Optional[int] = None, ws: Optional[GemmWorkspace] = None, push_comm=None,
             prefetch: Optional[QuantLinear] = None, cluster: Optional[bool] = None) -> torch.Tensor:
    """Block-scaled NVFP4 tensor-core linear on pre-quantised activations (token tile = xa.bn).
    splits > 1: split K.  cluster (default: on): the CTAs of one output tile form a thread-block cluster and fold
    their partial accumulators through distributed shared memory (no workspace); off: partials go through a global
    workspace and the last CTA of a tile folds them.
    prefetch: the projection that runs next; its packed weights are requested into L2 by this kernel's CTAs once
    their own loads are issued (fills the HBM-idle time of the small kernels in between; a hint, never needed).
    push_comm: native peer-communicator handle; the finished bf16 tiles are then stored into every rank's
    symmetric region (with per-tile flags) instead of `out` -- the first half of a fused all-reduce."""
    assert w.fmt == "nvfp4" and xa.k == w.k
    rows, bn = xa.rows, xa.bn
    dev = xa.q.device
    if out is None and out32 is None and not push_comm:
        out = torch.empty(rows, w.n, dtype=torch.bfloat16, device=dev)
    ldc = w.n if push_comm and out is None and out32 is None else (out if out is not None else out32).stride(0)
    if cluster is None:
        cluster = CLUSTER_SPLITK
    if splits is None:
        splits = pick_cluster_splits(rows, w.n, w.k, bn) if cluster else pick_splits_fp4(rows, w.n, w.k, bn)
    cluster = cluster and 2 <= splits <= 8 and (splits - 1) * bn * 512 <= 65536
    wsp = cnt = None
    if splits > 1 and not cluster:
        ws = ws or default_workspace(dev)
        if splits * rows * w.n > ws.partials.numel():
            splits = 1
        else:
            wsp, cnt = ws.partials, ws.counters
    if prefetch is not None:
        call("dgpp_gemm_fp4_set_prefetch", ptr(prefetch.payload), prefetch.payload.numel() // 16 * 16)
    call("dgpp_gemm_fp4", bn, ptr(xa.q), ptr(xa.sf), ptr(xa.g), xa.terms, xa.rows_pad, ptr(w.payload),
         ptr(w.tiled_scales()), float(w.alpha), ptr(out), ptr(out32), ptr(resid), ldc, rows, w.n, w.k, splits,
         ptr(wsp), ptr(cnt), push_comm, stream_ptr())
    return out if out is not None else out32


# Policies of the block-scaled GEMM, set by `configure` (from engine.options.EngineOptions; never from the environment).
CLUSTER_SPLITK = False


def configure(fp4_splits: Optional[str] = None, cluster_splitk: Optional[bool] = None,
              fp4_preload: Optional[bool] = None) -> None:
    """Process-wide GEMM policies: split-K policy ("auto" | "resident" | "legacy"), split-K through a thread-block
    cluster, and the pre-wait weight preload."""
    global CLUSTER_SPLITK, FP4_SPLIT_POLICY
    if fp4_splits is not None:
        assert fp4_splits in ("auto", "resident", "legacy")
        FP4_SPLIT_POLICY = fp4_splits
    if cluster_splitk is not None:
        CLUSTER_SPLITK = bool(cluster_splitk)
    if fp4_preload is not None and _lib.available() and torch.cuda.is_available():
        call("dgpp_gemm_fp4_set_preload", int(bool(fp4_preload)))


def pick_cluster_splits(rows: int, n: int, k: int, bn: int) -> int:
    """Cluster split-K for projections with few output tiles (decode qkv / o / down): a CTA that walks 20+ K stages
    alone is bound by the latency of its own scale-copy -> MMA -> commit chain, not by bandwidth; splitting K over the
    CTAs of a cluster shortens the chain and puts two CTAs on every SM.  At least 4 stages per CTA, cluster sizes 2 / 4 /
    8, and two to three resident CTAs per SM in total."""
    tiles = math.ceil(n / 128) * math.ceil(rows / bn)
    stages = k // 256
    if rows > 64 or tiles > 74 or stages < 8:
        return 1
    want = min(8, max(1, 444 // tiles), stages // 4)
    s = 1
    while s * 2 <= want and (s * 2 - 1) * bn * 512 <= 65536:      # cluster sizes 2 / 4 / 8
        s *= 2
    return s


# Split-K policy of the block-scaled GEMM in the weight-streaming regime.  "resident": split until one resident wave
# (two CTAs per SM) covers the problem, so that with the pre-wait weight preload most of a CTA's K range is already
# in its ring when the activations arrive; "legacy": split only long-K, few-tile problems.
# Measured on the 27B-class decode step: C8 7.14 ms legacy / 7.34 ms resident, C1 165.7 / 169.8 tok/s -- the fold's
# fences and counter round trip cost more than the shorter K range saves once 8 rows share the weights, so "auto"
# takes resident for a single row and legacy otherwise.
FP4_SPLIT_POLICY = "auto"


# True: the split-K choice of the block-scaled GEMM ignores whether a pass has one row or several, so a row computes the
# same bits in a plain decode pass and among speculative verify rows (set by speculation; the one-row tuning is lost).
PIN_SPLIT_ROWS = False


def pick_splits_fp4(rows: int, n: int, k: int, bn: int, sms: int = 148) -> int:
    """Split K for few-tile problems (the deterministic fold costs a few microseconds)."""
    if PIN_SPLIT_ROWS:
        rows = max(rows, 2)
    tiles = math.ceil(n / 128) * math.ceil(rows / bn)
    stages = k // 256
    if FP4_SPLIT_POLICY == "resident" or (FP4_SPLIT_POLICY == "auto" and rows == 1):
        if tiles > sms:
            return 1
        return max(1, min(2 * sms // tiles, stages // 2, 8))
    if tiles >= sms // 2 + 1 or stages <= 24:
        return 1 if (rows > 1 or tiles >= sms // 2 + 1) else max(1, min(3, stages // 4))
    return max(1, min(math.ceil(sms / tiles), stages // 8))


def linear(x: torch.Tensor, w: QuantLinear, out: Optional[torch.Tensor] = None,
           resid: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Dispatch a linear layer to the tensor-core kernel (all row counts)."""
    return gemm_tc(x, w, out=out, resid=resid)


def rope_kv_write(qkv, positions, row_req, block_table, inv_freq, cache, hq: int, hkv: int, d: int,
                  rot_dim: Optional[int] = None, mscale: float = 1.0, q_norm_w=None, k_norm_w=None,
                  eps: float = 1e-6, norm_one_plus_w: bool = False) -> None:
    """In-place RoPE on q/k of `qkv` and append of k/v into `cache` (a ``PagedKV`` layer view)."""
    _chk(qkv, torch.bfloat16, "qkv")
    rows = qkv.shape[0]
    call("dgpp_rope_kv_write", ptr(qkv), ptr(positions), ptr(row_req), ptr(block_table), ptr(inv_freq),
         ptr(q_norm_w), ptr(k_norm_w), ptr(cache.k), ptr(cache.v), ptr(cache.k_scale), ptr(cache.v_scale), rows,
         hq, hkv, d, rot_dim or d, cache.page, block_table.shape[1], float(mscale), float(eps), int(cache.fp8),
         int(norm_one_plus_w), stream_ptr())


def attn_decode(q, q_stride: int, cache, block_table, row_req, positions, hq: int, hkv: int, d: int,
                scale: float, splits: int = 1, scratch=None, out=None, window: int = 0, sink=None, sel=None,
                sel_block: int = 0):
    """CUDA-core decode attention over the paged cache (bf16 or FP8).  window > 0: sliding window; sink: optional
    [hq] fp32 logits of a value-less softmax column (sliding-window + sink attention families); sel: optional
    [rows, hkv, k] int32 ascending block ids of `sel_block` tokens (-1 padded, the row's own block last): every
    (row, kv head) then attends only to its listed blocks."""
    rows = positions.numel()
    if out is None:
        out = torch.empty(rows, hq * d, dtype=torch.bfloat16, device=positions.device)
    ml = acc = None
    if splits > 1:
        if scratch is None:
            scratch = (torch.empty(rows * hq * splits * 2, dtype=torch.float32, device=out.device),
                       torch.empty(rows * hq * splits * d, dtype=torch.float32, device=out.device))
        ml, acc = scratch
    if sel is not None:
        _chk(sel, torch.int32, "sel")
        assert sink is None and window == 0 and sel.shape[0] == rows and sel.shape[1] == hkv and sel_block > 0
        call("dgpp_attn_decode_sparse", ptr(q), q_stride, ptr(cache.k), ptr(cache.v), ptr(cache.k_scale),
             ptr(cache.v_scale), ptr(block_table), ptr(row_req), ptr(positions), ptr(ml), ptr(acc), ptr(out), rows, hq,
             hkv, d, cache.page, block_table.shape[1], splits, int(cache.fp8), float(scale), ptr(sel), sel.shape[2],
             sel_block, stream_ptr())
        return out
    if sink is not None:
        _chk(sink, torch.float32, "sink")
        assert sink.numel() == hq
        call("dgpp_attn_decode_sink", ptr(q), q_stride, ptr(cache.k), ptr(cache.v), ptr(cache.k_scale),
             ptr(cache.v_scale), ptr(block_table), ptr(row_req), ptr(positions), ptr(ml), ptr(acc), ptr(out), rows, hq,
             hkv, d, cache.page, block_table.shape[1], splits, int(cache.fp8), float(scale), window, ptr(sink),
             stream_ptr())
        return out
    call("dgpp_attn_decode", ptr(q), q_stride, ptr(cache.k), ptr(cache.v), ptr(cache.k_scale), ptr(cache.v_scale),
         ptr(block_table), ptr(row_req), ptr(positions), ptr(ml), ptr(acc), ptr(out), rows, hq, hkv, d, cache.page,
         block_table.shape[1], splits, int(cache.fp8), float(scale), window, stream_ptr())
    return out


def msa_index_prep(iqk, positions, row_req, block_table, inv_freq, q_norm_w, k_norm_w, index_cache, ih: int, di: int,
                   rot_dim: int, eps: float = 1e-6, one_plus_w: bool = False, raw_key: bool = False) -> None:
    """In place on iqk [rows, (ih + 1) * di] bf16 (index query heads, then the index key of the row): per-head RMSNorm
    and rotary embedding on the first rot_dim dims; the key is appended to index_cache [blocks, page, di] bf16.
    raw_key: the key is appended untouched (pooled-key form: blocks are compressed later by `qsa_compress`)."""
    _chk(iqk, torch.bfloat16, "iqk")
    _chk(index_cache, torch.bfloat16, "index_cache")
    assert iqk.shape[1] == (ih + 1) * di and iqk.is_contiguous() and index_cache.shape[2] == di
    call("dgpp_msa_index_prep", ptr(iqk), ptr(positions), ptr(row_req), ptr(block_table), ptr(inv_freq), ptr(q_norm_w),
         ptr(k_norm_w), ptr(index_cache), iqk.shape[0], ih, di, rot_dim, index_cache.shape[1], block_table.shape[1],
         float(eps), int(one_plus_w), int(raw_key), stream_ptr())


def qsa_compress(raw_cache, comp_cache, positions, row_req, block_table, inv_freq, k_norm_w, rot_dim: int,
                 eps: float = 1e-6, one_plus_w: bool = True) -> None:
    """For every row whose position completes a block of raw_cache [blocks, kpool, di] bf16: the block's keys averaged
    (fp32 mean, bf16), RMS-normalised and rotated at the block's first position -> comp_cache [blocks, di] bf16."""
    _chk(raw_cache, torch.bfloat16, "raw_cache")
    _chk(comp_cache, torch.bfloat16, "comp_cache")
    assert comp_cache.shape == (raw_cache.shape[0], raw_cache.shape[2])
    call("dgpp_qsa_compress", ptr(raw_cache), ptr(comp_cache), ptr(positions), ptr(row_req), ptr(block_table),
         ptr(inv_freq), ptr(k_norm_w), positions.numel(), raw_cache.shape[2], raw_cache.shape[1], rot_dim,
         block_table.shape[1], float(eps), int(one_plus_w), stream_ptr())


def qsa_select(iqk, comp_cache, block_table, row_req, positions, ih: int, di: int, kpool: int, select_k: int, max_sel: int,
               copies: int = 1, out=None, scores=None):
    """Pooled-key block selection -> int32 [rows, copies, select_k + 1]: ascending ids of the select_k complete visible
    blocks with the largest sum over index heads of relu(<q_h, compressed key>) / sqrt(di) (all of them when there
    are no more; ties to the lower id) plus the row's own incomplete block; -1 padded; the same list `copies` times
    (one per kv head for `attn_decode`)."""
    rows = positions.numel()
    if out is None:
        out = torch.empty(rows, copies, select_k + 1, dtype=torch.int32, device=positions.device)
    call("dgpp_qsa_select", ptr(iqk), iqk.stride(0), ptr(comp_cache), ptr(block_table), ptr(row_req), ptr(positions),
         ptr(out), ptr(scores), rows, ih, di, block_table.shape[1], kpool, select_k, max_sel, copies, stream_ptr())
    return out


def msa_index_select(iqk, index_cache, block_table, row_req, positions, ih: int, di: int, sel_block: int, topk: int,
                     max_sel: int, out=None, scores=None):
    """Block selection of block-sparse attention -> int32 [rows, ih, topk]: ascending ids of the `topk` blocks (of
    sel_block tokens) with the largest per-block maximum of <index query, index key> over the visible tokens, the
    row's own block always among them; -1 padded.  scores: fp32 [rows, ih, max_sel] workspace (the block scores stay
    there; allocated when not given: pass one inside captured passes)."""
    rows = positions.numel()
    if out is None:
        out = torch.empty(rows, ih, topk, dtype=torch.int32, device=positions.device)
    if scores is None:
        scores = torch.empty(rows, ih, max_sel, dtype=torch.float32, device=positions.device)
    call("dgpp_msa_index_select", ptr(iqk), iqk.stride(0), ptr(index_cache), ptr(block_table), ptr(row_req),
         ptr(positions), ptr(out), ptr(scores), rows, ih, di, index_cache.shape[1], block_table.shape[1], sel_block,
         topk, max_sel, stream_ptr())
    return out


def check_status() -> None:
    _lib.check_status()


_lib.declare("dgpp_segment_copy", [P, I, L, P])
_lib.declare("dgpp_stream_wait", [P, L])


def segment_copy(pairs) -> None:
    """One launch for many copies: pairs = [(src tensor, dst tensor), ...] of equal byte sizes per pair (multiples of 16,
    16-byte aligned).  The table goes to the device once per call; callers that repeat a set keep `segment_table`."""
    table, biggest = segment_table(pairs)
    call("dgpp_segment_copy", ptr(table), len(pairs), biggest, stream_ptr())


def segment_table(pairs):
    """Device table of (src, dst, bytes) records for dgpp_segment_copy; returns (table, largest segment in bytes)."""
    rec, biggest = [], 0
    for s, d in pairs:
        n = s.numel() * s.element_size()
        assert n == d.numel() * d.element_size() and n % 16 == 0 and s.is_contiguous() and d.is_contiguous()
        rec += [s.data_ptr(), d.data_ptr(), n]
        biggest = max(biggest, n)
    dev = pairs[0][0].device
    return torch.tensor(rec, dtype=torch.int64).to(dev), biggest


def stream_wait(timeout_s: float, stream=None) -> bool:
    """Bounded host wait for a stream: True when its work finished within the deadline, False when it is still pending
    (the caller decides: fail the engine, report); raises on a CUDA error."""
    rc = _lib._fn("dgpp_stream_wait")(stream_ptr(stream), int(timeout_s * 1e6))
    if rc < 0:
        raise RuntimeError("stream_wait: " + _lib.load().dgpp_last_error().decode())
    return rc == 0


def attn_decode_tc(q, q_stride: int, cache, block_table, row_req, positions, hq: int, hkv: int, d: int,
                   scale: float, splits: int = 1, scratch=None, out=None, window: int = 0,
                   partials_only: bool = False, sel=None, sel_block: int = 0):
    """Tensor-core (tcgen05, FP8 operands) decode attention over an FP8 paged cache; head_dim 128 or 256.
    partials_only (splits > 1): stop after the split-KV pass and leave the (max, sum) pairs and unnormalised
    accumulators in `scratch` for attn_combine_quant, which folds them while it quantises; returns None."""
    assert cache.fp8, "the tensor-core decode path reads e4m3 caches"
    rows = positions.numel()
    dev = positions.device
    if partials_only:
        assert splits > 1 and scratch is not None
        out = None
    elif out is None:
        out = torch.empty(rows, hq * d, dtype=torch.bfloat16, device=dev)
    ml = acc = None
    if splits > 1:
        if scratch is None:
            scratch = (torch.empty(rows * hq * splits * 2, dtype=torch.float32, device=dev),
                       torch.empty(rows * hq * splits * d, dtype=torch.float32, device=dev))
        ml, acc = scratch
    call("dgpp_attn_decode_tc", ptr(q), q_stride, ptr(cache.k), ptr(cache.v), ptr(cache.k_scale),
         ptr(cache.v_scale), ptr(block_table), ptr(row_req), ptr(positions), ptr(ml), ptr(acc), ptr(out), rows, hq,
         hkv, d, cache.page, block_table.shape[1], cache.k.shape[0], splits, float(scale), window, ptr(sel),
         0 if sel is None else sel.shape[2], sel_block, stream_ptr())
    return out


def attn_prefill_tc(q, q_stride: int, cache, block_table_row, pos0: int, hq: int, hkv: int, d: int, scale: float,
                    out=None, window: int = 0, rows: Optional[int] = None):
    """Causal tensor-core flash attention of a prefill chunk (rows at positions pos0.. of one request) against the
    FP8 paged cache that already holds those positions.  head_dim 128 or 256 (a kernel each)."""
    assert cache.fp8
    T = rows if rows is not None else q.shape[0]
    if out is None:
        out = torch.empty(T, hq * d, dtype=torch.bfloat16, device=q.device)
    call("dgpp_attn_prefill_tc256" if d == 256 else "dgpp_attn_prefill_tc", ptr(q), q_stride, ptr(cache.k), ptr(cache.v), ptr(cache.k_scale), ptr(cache.v_scale),
         ptr(block_table_row), ptr(out), T, pos0, hq, hkv, d, cache.page, block_table_row.numel(), cache.k.shape[0],
         float(scale), window, stream_ptr())
    return out


# ---------------------------------------------------------------------------------------------- vision tower
def vis_patchify(canvas: torch.Tensor, out: torch.Tensor, patch: int, merge: int, mean, std) -> torch.Tensor:
    """uint8 canvas [H, W, 3] -> normalised bf16 patch rows [patches, 3 * patch^2] (merge groups contiguous)."""
    import ctypes
    assert canvas.dtype == torch.uint8 and canvas.is_contiguous() and out.is_contiguous()
    H, W, _ = canvas.shape
    m3, s3 = (ctypes.c_float * 3)(*mean), (ctypes.c_float * 3)(*std)
    call("dgpp_vis_patchify", ptr(canvas), ptr(out), H, W, patch, merge, ctypes.addressof(m3), ctypes.addressof(s3),
         stream_ptr())
    return out


def layernorm(x: torch.Tensor, w: torch.Tensor, b: Optional[torch.Tensor], eps: float = 1e-6,
              out: Optional[torch.Tensor] = None) -> torch.Tensor:
    _chk(x, torch.bfloat16, "x")
    assert x.is_contiguous()
    if out is None:
        out = torch.empty_like(x)
    call("dgpp_layernorm", ptr(x), ptr(w), ptr(b), ptr(out), x.shape[0], x.shape[1], float(eps), stream_ptr())
    return out


def bias_act(x: torch.Tensor, bias: Optional[torch.Tensor], resid: Optional[torch.Tensor] = None, act: int = 0):
    """In place: x = resid + act(x + bias); act 0 none, 1 GELU (erf), 2 GELU (tanh)."""
    _chk(x, torch.bfloat16, "x")
    assert x.is_contiguous() and (resid is None or resid.is_contiguous())
    call("dgpp_bias_act", ptr(x), ptr(bias), ptr(resid), x.shape[0], x.shape[1], act, stream_ptr())
    return x


def vis_qkv_split_rope(qkv, bias, pos_y, pos_x, q_h, k_h, vt_h, heads: int, d: int, theta: float) -> None:
    """[T, 3 * heads * d] -> head-major q / k with 2-D RoPE and V transposed [heads, d, T_pad]."""
    T = qkv.shape[0]
    call("dgpp_vis_qkv_split_rope", ptr(qkv), ptr(bias), ptr(pos_y), ptr(pos_x), ptr(q_h), ptr(k_h), ptr(vt_h), T,
         vt_h.shape[2], heads, d, float(theta), stream_ptr())


def softmax_rows(s: torch.Tensor, cols: int) -> torch.Tensor:
    """In-place softmax over the first `cols` columns of every row of the bf16 matrix s; the rest becomes zero."""
    _chk(s, torch.bfloat16, "s")
    call("dgpp_softmax_rows", ptr(s), s.shape[0], cols, s.stride(0), stream_ptr())
    return s


# ---------------------------------------------------------------------------------------------- mixture of experts
from ._lib import F, I, L, P  # noqa: E402  (ctypes aliases for the signatures below)

_lib.declare("dgpp_moe_route", [P, L, P, P, P, P, P, I, I, I, I, I, I, I, I, F, P])
_lib.declare("dgpp_moe_active", [P, I, I, I, I, P, P, P, I, I, P])
_lib.declare("dgpp_moe_combine_push", [P, P, P, P, P, P, I, I, I, I, P])
_lib.declare("dgpp_moe_combine", [P, P, P, P, P, P, I, I, I, I, P])
_lib.declare("dgpp_gemm_fp4_grouped", [I, P, P, P, I, P, P, P, P, I, L, I, I, I, I, I, P, I, I, P, P, P])


def moe_route(x, gate, bias, k: int, n_group: int = 1, topk_group: int = 1, softmax: bool = False,
              norm_topk: bool = True, scaling: float = 1.0, ids=None, weights=None, logits_out=None):
    """Router: x [T, H] bf16, gate [E, H] bf16, bias [E] fp32 or None -> (ids [T, k] int32 ascending, weights [T, k])."""
    T, H = x.shape
    E = gate.shape[0]
    if ids is None:
        ids = torch.empty(T, k, dtype=torch.int32, device=x.device)
        weights = torch.empty(T, k, dtype=torch.float32, device=x.device)
    if logits_out is None:
        logits_out = torch.empty(T, E, dtype=torch.float32, device=x.device)
    call("dgpp_moe_route", ptr(x), x.stride(0), ptr(gate), ptr(bias), ptr(ids), ptr(weights), ptr(logits_out), T, H, E, k,
         n_group, topk_group, int(softmax), int(norm_topk), float(scaling), stream_ptr())
    return ids, weights


def moe_active(ids, rows: int, experts: int, slots: int, group_list=None, slot_of=None, n_active=None,
               e_begin: int = 0, e_end: int = 0):
    """Active-expert list.  With expert parallelism only experts [e_begin, e_end) are listed (as local indices)."""
    dev = ids.device
    if group_list is None:
        group_list = torch.empty(slots, dtype=torch.int32, device=dev)
        slot_of = torch.empty(experts, dtype=torch.int32, device=dev)
        n_active = torch.empty(1, dtype=torch.int32, device=dev)
    call("dgpp_moe_active", ptr(ids), rows, ids.shape[1], experts, slots, ptr(group_list), ptr(slot_of), ptr(n_active),
         e_begin, e_end, stream_ptr())
    return group_list, slot_of, n_active


def moe_combine(y, shared, ids, weights, slot_of, out, rows: int):
    """y [slots, rows_per_slot, H]; out[t] = sum_j w[t, j] * y[slot_of[ids[t, j]], t] (+ shared[t])."""
    call("dgpp_moe_combine", ptr(y), ptr(shared), ptr(ids), ptr(weights), ptr(slot_of), ptr(out), rows, y.shape[2],
         ids.shape[1], y.shape[1], stream_ptr())
    return out


def moe_combine_push(y, shared, ids, weights, slot_of, comm, rows: int):
    """Expert-parallel combine: this rank's partial is pushed to every rank's symmetric region (consumed by the
    fold in the next add + RMSNorm + quantise kernel)."""
    call("dgpp_moe_combine_push", ptr(y), ptr(shared), ptr(ids), ptr(weights), ptr(slot_of), comm, rows, y.shape[2],
         ids.shape[1], y.shape[1], stream_ptr())


_lib.declare("dgpp_moe_segment_sort", [P, P, P, P, I, I, I, I, I, I, P])
_lib.declare("dgpp_moe_gather_rows", [P, L, P, P, I, I, I, P])
_lib.declare("dgpp_moe_combine_rows", [P, P, P, P, P, I, I, I, P])


def moe_segment_sort(ids, bn: int, max_tiles: int, e_begin: int, e_end: int, pair_row=None, tile_expert=None, n_tiles=None):
    """Counting sort of the (token, k) pairs of `ids` [T, k] by local expert into tiles of bn rows (stable: pairs keep
    their order inside an expert).  Returns pair_row [T * k] (row of the pair in the tiled buffer, -1 if its expert is
    not in [e_begin, e_end)), tile_expert [max_tiles] (local expert id per tile, -1 beyond the last), n_tiles [1]."""
    T, k = ids.shape
    dev = ids.device
    if pair_row is None:
        pair_row = torch.empty(T * k, dtype=torch.int32, device=dev)
        tile_expert = torch.empty(max_tiles, dtype=torch.int32, device=dev)
        n_tiles = torch.empty(1, dtype=torch.int32, device=dev)
    call("dgpp_moe_segment_sort", ptr(ids), ptr(pair_row), ptr(tile_expert), ptr(n_tiles), T, k, e_begin, e_end, bn,
         max_tiles, stream_ptr())
    return pair_row, tile_expert, n_tiles


def moe_gather_rows(x, pair_row, xs, k: int):
    """xs[pair_row[p]] = x[p // k] for every pair with a row."""
    call("dgpp_moe_gather_rows", ptr(x), x.stride(0), ptr(pair_row), ptr(xs), x.shape[0], x.shape[1], k, stream_ptr())
    return xs


def moe_combine_rows(y, shared, pair_row, weights, out):
    """out[t] = sum_j weights[t, j] * y[pair_row[t * k + j]] (+ shared[t]); y: [rows, H] bf16."""
    T, k = weights.shape
    call("dgpp_moe_combine_rows", ptr(y), ptr(shared), ptr(pair_row), ptr(weights), ptr(out), T, y.shape[-1], k, stream_ptr())
    return out


def gemm_fp4_grouped(xa: "QuantAct", wq, wsf_tiled, alphas, out, rows: int, n: int, k: int, experts: int, group_list,
                     group_b: bool, splits: int = 1, ws: Optional["GemmWorkspace"] = None):
    """Grouped block-scaled NVFP4 GEMM over stacked expert matrices (see dgpp_gemm_fp4_grouped).
    out: [slots, bn, n] bf16 (row stride n)."""
    slots = group_list.numel()
    wsp = cnt = None
    if splits > 1:
        ws = ws or default_workspace(xa.q.device)
        if splits * rows * slots * n > ws.partials.numel() or slots * (n // 128) > ws.counters.numel():
            splits = 1
        else:
            wsp, cnt = ws.partials, ws.counters
    call("dgpp_gemm_fp4_grouped", xa.bn, ptr(xa.q), ptr(xa.sf), ptr(xa.g), xa.terms, ptr(wq), ptr(wsf_tiled), ptr(alphas),
         ptr(out), out.stride(1), out.stride(0), rows, n, k, experts, slots, ptr(group_list), int(group_b), splits,
         ptr(wsp), ptr(cnt), stream_ptr())
    return out


# ---------------------------------------------------------------------------------------------- table routing, Hadamard-32
_lib.declare("dgpp_moe_hash_routes", [P, P, P, P, P, I, I, I, I, F, I, P])
_lib.declare("dgpp_hadamard32_rows", [P, L, P, L, I, I, I, P])
_lib.declare("dgpp_hadamard32_quant_int8", [P, L, P, L, P, L, I, I, I, P])


def moe_hash_routes(tokens, tid2eid, scores, scaling: float = 1.0, norm_topk: bool = True):
    """Table routing: ids[t] = tid2eid[tokens[t]] ([vocab, k] int32, ascending per row), weights from `scores` [T, E] fp32."""
    T, E = scores.shape
    vocab, k = tid2eid.shape
    ids = torch.empty(T, k, dtype=torch.int32, device=scores.device)
    w = torch.empty(T, k, dtype=torch.float32, device=scores.device)
    call("dgpp_moe_hash_routes", ptr(tokens), ptr(tid2eid), ptr(scores), ptr(ids), ptr(w), T, vocab, E, k, float(scaling),
         int(norm_topk), stream_ptr())
    return ids, w


_lib.declare("dgpp_ple_embed_add", [P, P, P, P, I, I, I, P])


def ple_embed_add(tokens: torch.Tensor, prev: torch.Tensor, table: torch.Tensor, x: torch.Tensor) -> torch.Tensor:
    """Hashed bigram embeddings, in place: x[r] += table[(prev[r] * 1000003 + tokens[r] * 7919 + 12345) % len(table)]."""
    _chk(tokens, torch.int32, "tokens")
    _chk(prev, torch.int32, "prev")
    _chk(table, torch.bfloat16, "table")
    _chk(x, torch.bfloat16, "x")
    call("dgpp_ple_embed_add", ptr(tokens), ptr(prev), ptr(table), ptr(x), x.shape[0], x.shape[1], table.shape[0], stream_ptr())
    return x


def engram_embed(tokens, prev, token_map, multipliers, primes, offsets, table, table_sf, pad_class: int, out=None,
                 ids=None):
    """Hashed n-gram memory lookup: tokens [rows] and prev [max_ngram - 1, rows] int32 (row k: the token k + 1 positions
    back, -1 before the start) -> bf16 [rows, (max_ngram - 1) * heads * D] dequantised table rows.  multipliers
    [max_ngram], primes / offsets [max_ngram - 1, heads] int64; table [rows, D] e4m3 bytes, table_sf [rows, D / 32]
    e8m0 bytes.  ids: optional int32 [rows, (max_ngram - 1) * heads] out."""
    rows, max_ngram = tokens.numel(), multipliers.numel()
    heads, d = primes.shape[1], table.shape[1]
    assert prev.shape == (max_ngram - 1, rows) and prev.is_contiguous() and primes.shape == offsets.shape == (max_ngram - 1, heads)
    assert multipliers.dtype == primes.dtype == offsets.dtype == torch.int64 and table.dtype == table_sf.dtype == torch.uint8
    if out is None:
        out = torch.empty(rows, (max_ngram - 1) * heads * d, dtype=torch.bfloat16, device=tokens.device)
    call("dgpp_engram_embed", ptr(tokens), ptr(prev), ptr(token_map), ptr(multipliers), ptr(primes), ptr(offsets),
         ptr(table), ptr(table_sf), ptr(out), ptr(ids), rows, max_ngram, heads, d, int(pad_class), token_map.numel(),
         table.shape[0], stream_ptr())
    return out


def engram_gate(streams, kv, q_weight, k_weight, eps: float = 1e-6):
    """streams [rows, hc, H] bf16 in place: stream i takes the value of kv [rows, (hc + 1) * H] (keys, then the value)
    in through sigmoid(signed sqrt of its normalised weighted dot with key i)."""
    _chk(streams, torch.bfloat16, "streams")
    _chk(kv, torch.bfloat16, "kv")
    rows, hc, h = streams.shape
    assert kv.shape == (rows, (hc + 1) * h) and kv.is_contiguous() and streams.is_contiguous()
    call("dgpp_engram_gate", ptr(streams), ptr(kv), ptr(q_weight), ptr(k_weight), rows, hc, h, float(eps), stream_ptr())
    return streams


def hadamard32_rows(x: torch.Tensor, out: Optional[torch.Tensor] = None, period: int = 0) -> torch.Tensor:
    """Normalised block-32 Walsh-Hadamard rotation of bf16 rows (in place when out is x); rows r with
    r % period == period - 1 are not touched (period 0: all rows)."""
    _chk(x, torch.bfloat16, "x")
    if out is None:
        out = torch.empty_like(x) if period == 0 else x.clone()
    call("dgpp_hadamard32_rows", ptr(x), x.stride(0), ptr(out), out.stride(0), x.shape[0], x.shape[1], period, stream_ptr())
    return out


def hadamard32_quant_int8(x: torch.Tensor, period: int = 0):
    """Rotated rows as int8 codes [rows, K] + fp32 scales [rows, K / 128] (skipped rows keep zeros)."""
    _chk(x, torch.bfloat16, "x")
    rows, k = x.shape
    codes = torch.zeros(rows, k, dtype=torch.int8, device=x.device)
    scales = torch.zeros(rows, k // 128, dtype=torch.float32, device=x.device)
    call("dgpp_hadamard32_quant_int8", ptr(x), x.stride(0), ptr(codes), codes.stride(0), ptr(scales), scales.stride(0), rows, k,
         period, stream_ptr())
    return codes, scales


# ---------------------------------------------------------------------------------------------- family operators
_lib.declare("dgpp_justnorm", [P, P, I, I, F, P])
_lib.declare("dgpp_slerp_alpha", [P, P, P, F, P, I, I, F, P])
_lib.declare("dgpp_gr_gate_act", [P, L, I, I, P])
_lib.declare("dgpp_gr_mix_finish", [P, P, P, I, I, I, P])
_lib.declare("dgpp_gr_combine", [P, P, P, P, P, I, I, I, P])


def justnorm(x: torch.Tensor, eps: float = 1e-6) -> torch.Tensor:
    """Unit-norm rows: bf16(x / sqrt(sum x^2 + eps)), the sum in fp64."""
    _chk(x, torch.bfloat16, "x")
    y = torch.empty_like(x)
    call("dgpp_justnorm", ptr(x), ptr(y), x.shape[0], x.shape[1], float(eps), stream_ptr())
    return y


def slerp_alpha(a: torch.Tensor, b: torch.Tensor, alpha: torch.Tensor, s: float, eps: float = 1e-6) -> torch.Tensor:
    """Hypersphere residual: justnorm(an + |alpha s| (bn - an)) with an / bn the bf16 unit-norm rows of a / b."""
    _chk(a, torch.bfloat16, "a")
    _chk(b, torch.bfloat16, "b")
    _chk(alpha, torch.bfloat16, "alpha")
    out = torch.empty_like(a)
    call("dgpp_slerp_alpha", ptr(a), ptr(b), ptr(alpha), float(s), ptr(out), a.shape[0], a.shape[1], float(eps), stream_ptr())
    return out


def gr_gate_act(t: torch.Tensor, hc: int) -> torch.Tensor:
    """In place: t = bf16(silu(bf16(t / hc)))."""
    call("dgpp_gr_gate_act", ptr(t), t.shape[0], t.shape[1], hc, stream_ptr())
    return t


def gr_mix_finish(logits: torch.Tensor, rn: torch.Tensor, hc: int) -> torch.Tensor:
    """logits, rn [rows, hc * H] -> x [rows, H]: gated mean over the hc branches."""
    rows, H = logits.shape[0], logits.shape[1] // hc
    x = torch.empty(rows, H, dtype=torch.bfloat16, device=logits.device)
    call("dgpp_gr_mix_finish", ptr(logits), ptr(rn), ptr(x), rows, hc, H, stream_ptr())
    return x


def gr_combine(r_state: torch.Tensor, rn: torch.Tensor, w_inject: torch.Tensor, y: torch.Tensor, hc: int, gates=None) -> torch.Tensor:
    """In place on r_state [rows, hc * H]: branch i += bf16(y * s_i), s_i = 2 sigmoid(<w_inject[i], rn[row]> / hc)."""
    rows, H = y.shape
    call("dgpp_gr_combine", ptr(r_state), ptr(rn), ptr(w_inject), ptr(y), ptr(gates), rows, hc, H, stream_ptr())
    return r_state


_lib.declare("dgpp_mhc_compute", [P, P, P, P, P, P, P, I, I, I, I, F, F, P])
_lib.declare("dgpp_mhc_fold", [P, P, P, P, P, I, I, I, P])


def mhc_compute(streams, fn, base, scale, iters: int = 20, hc_eps: float = 1e-6, norm_eps: float = 1e-5):
    """Hyper-connection coefficients of n residual streams [tokens, n, D]: returns (collapsed [tokens, D], post [tokens, n],
    comb [tokens, n, n]) in bf16.  fn: bf16 [(2 + n) n, n D]; base fp32 [(2 + n) n]; scale fp32 [3]."""
    tokens, n, D = streams.shape
    dev = streams.device
    collapsed = torch.empty(tokens, D, dtype=torch.bfloat16, device=dev)
    post = torch.empty(tokens, n, dtype=torch.bfloat16, device=dev)
    comb = torch.empty(tokens, n, n, dtype=torch.bfloat16, device=dev)
    call("dgpp_mhc_compute", ptr(streams), ptr(fn), ptr(base), ptr(scale), ptr(collapsed), ptr(post), ptr(comb), tokens, n, D,
         iters, float(hc_eps), float(norm_eps), stream_ptr())
    return collapsed, post, comb


def mhc_fold(streams, h, post, comb, out=None):
    """streams'[i] = bf16(bf16(post_i h) + bf16(sum_j comb[j, i] streams[j])); out may be `streams` (in place)."""
    tokens, n, D = streams.shape
    if out is None:
        out = torch.empty_like(streams)
    call("dgpp_mhc_fold", ptr(streams), ptr(h), ptr(post), ptr(comb), ptr(out), tokens, n, D, stream_ptr())
    return out


# ---------------------------------------------------------------------------------------------- native FP8 linear
_lib.declare("dgpp_fp8_act_quant", [P, L, P, P, I, I, I, P])
_lib.declare("dgpp_gemm_fp8", [P, P, P, P, P, P, I, I, I, I, I, I, I, P])


class Fp8Act:
    """Activations as e4m3 bytes [rows_pad, K] with one fp32 scale per token and 128 columns (stored [K / 128, rows_pad])."""

    def __init__(self, rows_pad: int, k: int, device):
        self.q = torch.zeros(rows_pad, k, dtype=torch.uint8, device=device)
        self.scale = torch.ones(k // 128, rows_pad, dtype=torch.float32, device=device)
        self.rows, self.rows_pad, self.k = 0, rows_pad, k

    def dequant(self) -> torch.Tensor:
        v = self.q[:self.rows].view(torch.float8_e4m3fn).float().view(self.rows, self.k // 128, 128)
        return (v * self.scale[:, :self.rows].t().unsqueeze(-1)).reshape(self.rows, self.k)


def fp8_act_quant(x: torch.Tensor, out: Optional[Fp8Act] = None, bn: Optional[int] = None) -> Fp8Act:
    """Per-token, per-128-column e4m3 quantisation of bf16 rows (scale = amax / 448)."""
    _chk(x, torch.bfloat16, "x")
    rows, k = x.shape
    if out is None:
        bn = bn or min(pick_bn(rows), 128)
        out = Fp8Act((rows + bn - 1) // bn * bn, k, x.device)
    assert rows <= out.rows_pad and out.k == k
    out.rows = rows
    call("dgpp_fp8_act_quant", ptr(x), x.stride(0), ptr(out.q), ptr(out.scale), rows, out.rows_pad, k, stream_ptr())
    return out


def gemm_fp8(xa: Fp8Act, w: QuantLinear, out: Optional[torch.Tensor] = None, splits: Optional[int] = None) -> torch.Tensor:
    """Block-scaled FP8 weights (128 x 128 blocks) x FP8 activations on tcgen05 kind::f8f6f4, scales promoted per K block."""
    assert w.fmt == "fp8" and xa.k == w.k and w.alpha == 1.0
    rows = xa.rows
    bn = min(pick_bn(rows), 128)
    while xa.rows_pad % bn:
        bn //= 2
    if out is None:
        out = torch.empty(rows, w.n, dtype=torch.bfloat16, device=xa.q.device)
    if splits is None:
        tiles = math.ceil(w.n / 128) * math.ceil(rows / bn)
        splits = 1 if (tiles >= 96 or rows > 128) else max(1, min(148 // tiles, (w.k // 128) // 4, 8))
    partial = None
    if splits > 1:
        partial = torch.empty(splits * rows * w.n, dtype=torch.float32, device=xa.q.device)
    call("dgpp_gemm_fp8", ptr(w.payload), ptr(w.scale), ptr(xa.q), ptr(xa.scale), ptr(out), ptr(partial), out.stride(0), rows,
         xa.rows_pad, w.n, w.k, bn, splits, stream_ptr())
    return out


def linear_fp8(x: torch.Tensor, w: QuantLinear, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """FP8 linear end to end: quantise the rows, run the native FP8 GEMM."""
    return gemm_fp8(fp8_act_quant(x), w, out=out)


# ---------------------------------------------------------------------------------------------- gated delta net
_lib.declare("dgpp_gdn_recurrent", [P, L, P, L, P, L, P, P, L, P, P, P, P, I, P, P, I, I, I, I, I, I, P])
_lib.declare("dgpp_gdn_conv", [P, L, P, P, P, P, I, P, I, I, I, I, P])
_lib.declare("dgpp_gated_rmsnorm", [P, P, L, P, P, I, I, I, F, P])


_lib.declare("dgpp_gdn_recurrent_runs", [P, L, P, L, P, L, P, P, L, P, P, P, P, P, P, I, I, I, I, I, I, P, P])
_lib.declare("dgpp_gdn_conv_runs", [P, L, P, P, P, P, P, I, I, I, I, P, P])
_lib.declare("dgpp_spec_accept", [P, P, P, P, I, I, P])
_lib.declare("dgpp_spec_commit", [P, P, P, P, P, P, I, I, I, I, I, L, L, P])
_lib.declare("dgpp_gdn_prep", [P, L, P, L, P, P, L, P, P, P, I, I, I, I, P])
_lib.declare("dgpp_gdn_chunk_scan", [P, P, P, P, P, L, P, P, P, L, I, I, I, I, I, P])
# Sequential runs of at least this many rows take the chunked scan; shorter ones (and decode) the token recurrence.
GDN_CHUNKED = True
GDN_CHUNK_MIN_ROWS = 64
_GDN_SCRATCH: dict = {}


def _gdn_scratch(device, floats: int) -> torch.Tensor:
    """Scratch of the chunked scan (W, U0, P, G per chunk and head), grown on demand and kept per device."""
    key = str(device)
    t = _GDN_SCRATCH.get(key)
    if t is None or t.numel() < floats:
        t = torch.empty(floats, dtype=torch.float32, device=device)
        _GDN_SCRATCH[key] = t
    return t


def gdn_conv(x, w, bias, state, out, row_slot=None, slot: int = 0, sequential: bool = True, seg: int = 0, snap=None):
    """Causal depthwise conv (width w.shape[1]) + SiLU.  x: [T, C] bf16 rows (may be a strided column view);
    state: [slots, W - 1, C] fp32, updated in place.  seg > 0: the rows are runs of `seg` consecutive tokens, run r
    belonging to slot row_slot[r * seg]; snap [T, W - 1, C] (optional) receives the tail after every row."""
    T, C = x.shape
    if seg > 0:
        call("dgpp_gdn_conv_runs", ptr(x), x.stride(0), ptr(w), ptr(bias), ptr(state), ptr(row_slot), ptr(out), T, C,
             w.shape[1], seg, ptr(snap), stream_ptr())
        return out
    call("dgpp_gdn_conv", ptr(x), x.stride(0), ptr(w), ptr(bias), ptr(state), ptr(row_slot), slot, ptr(out), T, C,
         w.shape[1], int(sequential), stream_ptr())
    return out


def gdn_recurrent(q, k, v, alpha, beta, A_log, dt_bias, state, out, hk: int, hv: int, dk: int, dv: int, row_slot=None,
                  slot: int = 0, sequential: bool = True, prep=None, seg: int = 0, snap=None):
    """Gated delta-rule recurrence.  q/k: [T, hk*dk], v: [T, hv*dv] (column views allowed), alpha/beta: [T, hv]
    views with a common row stride; state [slots, hv, dk, dv] fp32 updated in place; out [T, hv*dv] bf16.
    seg > 0: runs of `seg` consecutive tokens per request (slot row_slot[r * seg]); snap [T, hv, dk, dv] (optional)
    receives the state after every row."""
    T = q.shape[0]
    assert alpha.stride(0) == beta.stride(0)
    need = T * (2 * hk * dk + 2 * hv)
    if prep is None or prep.numel() < need:
        prep = torch.empty(need, dtype=torch.float32, device=q.device)
    if seg > 0:
        call("dgpp_gdn_recurrent_runs", ptr(q), q.stride(0), ptr(k), k.stride(0), ptr(v), v.stride(0), ptr(alpha), ptr(beta),
             alpha.stride(0), ptr(A_log), ptr(dt_bias), ptr(state), ptr(row_slot), ptr(out), ptr(prep), T, hk, hv, dk, dv,
             seg, ptr(snap), stream_ptr())
        return out
    if sequential and GDN_CHUNKED and T >= GDN_CHUNK_MIN_ROWS and dk in (64, 128) and dv % 32 == 0:
        # prefill: chunked scan (64-token chunks as small GEMMs) instead of T dependent token steps
        chunks = (T + 63) // 64
        floats = chunks * hv * 64 * (dk + dv + 65)
        scr = _gdn_scratch(q.device, floats)
        call("dgpp_gdn_prep", ptr(q), q.stride(0), ptr(k), k.stride(0), ptr(alpha), ptr(beta), alpha.stride(0),
             ptr(A_log), ptr(dt_bias), ptr(prep), T, hk, hv, dk, stream_ptr())
        qn, kn = prep, prep[T * hk * dk:]
        dec = prep[2 * T * hk * dk:]
        bet = dec[T * hv:]
        call("dgpp_gdn_chunk_scan", ptr(qn), ptr(kn), ptr(dec), ptr(bet), ptr(v), v.stride(0), ptr(state[slot]), ptr(out),
             ptr(scr), scr.numel(), T, hk, hv, dk, dv, stream_ptr())
        return out
    call("dgpp_gdn_recurrent", ptr(q), q.stride(0), ptr(k), k.stride(0), ptr(v), v.stride(0), ptr(alpha), ptr(beta),
         alpha.stride(0), ptr(A_log), ptr(dt_bias), ptr(state), ptr(row_slot), slot, ptr(out), ptr(prep), T, hk, hv, dk,
         dv, int(sequential), stream_ptr())
    return out


_lib.declare("dgpp_kda_recurrent", [P, L, P, L, P, L, P, L, P, L, P, P, F, P, P, I, P, P, I, I, I, I, I, I, I, P, P])


def kda_recurrent(q, k, v, gate, beta, A_log, dt_bias, lower_bound: float, state, out, hk: int, hv: int, dk: int, dv: int,
                  row_slot=None, slot: int = 0, sequential: bool = True, seg: int = 0, snap=None, prep=None):
    """Delta-rule recurrence with per-channel decay (KDA): gate [T, hv * dk] raw gate rows, beta [T, hv] raw write
    strengths, dt_bias [hv * dk]; decay of channel c = exp(lower_bound / (1 + exp(-exp(A_log[h]) (gate + dt_bias)))).
    state [slots, hv, dk, dv] fp32 in place; out [T, hv * dv] bf16.  Rows / runs / snapshots as in gdn_recurrent."""
    T = q.shape[0]
    need = T * (2 * hk * dk + 2 * hv + hv * dk)
    if prep is None or prep.numel() < need:
        prep = torch.empty(need, dtype=torch.float32, device=q.device)
    call("dgpp_kda_recurrent", ptr(q), q.stride(0), ptr(k), k.stride(0), ptr(v), v.stride(0), ptr(gate), gate.stride(0),
         ptr(beta), beta.stride(0), ptr(A_log), ptr(dt_bias), float(lower_bound), ptr(state), ptr(row_slot), slot, ptr(out),
         ptr(prep), T, hk, hv, dk, dv, int(sequential), seg, ptr(snap), stream_ptr())
    return out


def spec_accept(tokens, picks, n_acc, emitted, runs: int, run_rows: int) -> None:
    """Greedy verdict of speculative runs: tokens / picks [runs * run_rows] int32 -> n_acc [runs], emitted [runs, run_rows]."""
    call("dgpp_spec_accept", ptr(tokens), ptr(picks), ptr(n_acc), ptr(emitted), runs, run_rows, stream_ptr())


def spec_commit(ssm, ssm_snap, conv, conv_snap, run_slot, n_acc, runs: int, run_rows: int) -> None:
    """Roll the recurrent state of partially accepted runs back to the snapshot after their last kept row.
    ssm [layers, slots, ...] / ssm_snap [layers, rows, ...] fp32 (same for the convolution tails)."""
    layers, slots = ssm.shape[0], ssm.shape[1]
    rows = ssm_snap.shape[1]
    S = ssm[0, 0].numel()
    Cc = conv[0, 0].numel()
    call("dgpp_spec_commit", ptr(ssm), ptr(ssm_snap), ptr(conv), ptr(conv_snap), ptr(run_slot), ptr(n_acc), layers, slots,
         rows, runs, run_rows, S, Cc, stream_ptr())


def gated_rmsnorm(o, z, w, out, heads: int, d: int, eps: float = 1e-6):
    """out = rmsnorm(o per head) * w * silu(z); o/out: [rows, heads*d] contiguous, z: [rows, heads*d] view."""
    call("dgpp_gated_rmsnorm", ptr(o), ptr(z), z.stride(0), ptr(w), ptr(out), o.shape[0], heads, d, float(eps), stream_ptr())
    return out


# ---------------------------------------------------------------------------------------------- latent attention
_lib.declare("dgpp_mla_decode", [P, P, P, P, P, P, I, P, P, P, I, I, I, I, I, I, I, F, P])
_lib.declare("dgpp_mla_decode_tc", [P, P, P, P, P, P, I, P, P, P, I, I, I, I, I, I, I, I, F, P])
_lib.declare("dgpp_dsa_index", [P, P, P, P, P, P, P, I, I, I, I, I, I, P])
_lib.declare("dgpp_topk_select", [P, L, P, P, I, I, P])


def mla_decode(q, cache, block_table, row_req, positions, scale: float, dc: int, dr: int, sel=None, splits: int = 1,
               out=None, tensor_cores: Optional[bool] = None):
    """Absorbed multi-head latent attention.  q: [rows, heads, dc + dr] bf16; cache: [blocks, page, dc + dr] bf16;
    sel: optional [rows, n_sel] int32 selected token positions (ascending, -1 padded) for sparse attention.
    Returns the latent outputs [rows, heads, dc] bf16.  The 512 + 64 geometry runs on the tensor cores, dense or sparse
    (tensor_cores=False keeps the CUDA-core kernel)."""
    rows, heads, _ = q.shape
    dev = q.device
    if out is None:
        out = torch.empty(rows, heads, dc, dtype=torch.bfloat16, device=dev)
    ml = acc = None
    if splits > 1:
        ml = torch.empty(rows * heads * splits * 2, dtype=torch.float32, device=dev)
        acc = torch.empty(rows * heads * splits * dc, dtype=torch.float32, device=dev)
    if tensor_cores is None:
        tensor_cores = dc == 512 and dr == 64 and cache.shape[1] in (16, 32, 64, 128)
    if tensor_cores:
        call("dgpp_mla_decode_tc", ptr(q), ptr(cache), ptr(block_table), ptr(row_req), ptr(positions), ptr(sel),
             0 if sel is None else sel.shape[1], ptr(ml), ptr(acc), ptr(out), rows, heads, dc, dr, cache.shape[1],
             block_table.shape[1], cache.shape[0], splits, float(scale), stream_ptr())
        return out
    call("dgpp_mla_decode", ptr(q), ptr(cache), ptr(block_table), ptr(row_req), ptr(positions), ptr(sel),
         0 if sel is None else sel.shape[1], ptr(ml), ptr(acc), ptr(out), rows, heads, dc, dr, cache.shape[1],
         block_table.shape[1], splits, float(scale), stream_ptr())
    return out


_lib.declare("dgpp_mla_kv_prep", [P, L, P, F, P, P, P, P, I, I, P, I, I, I, P])
_lib.declare("dgpp_mla_q_absorb", [P, P, P, P, P, I, I, I, I, I, P])
_lib.declare("dgpp_mla_v_up", [P, P, P, I, I, I, I, P])


def mla_kv_prep(kv, norm_w, eps: float, inv_freq, positions, row_req, block_table, cache, dc: int, dr: int) -> None:
    """kv [rows, dc + dr] bf16 (projection output): RMSNorm of the latent part, RoPE of the rotary key, both written to
    the rows' slots of the paged latent cache [blocks, page, dc + dr]."""
    call("dgpp_mla_kv_prep", ptr(kv), kv.stride(0), ptr(norm_w), float(eps), ptr(inv_freq), ptr(positions), ptr(row_req),
         ptr(block_table), block_table.shape[1], cache.shape[1], ptr(cache), kv.shape[0], dc, dr, stream_ptr())


def mla_q_absorb(q, w_uk, inv_freq, positions, dc: int, dr: int, out=None):
    """q [rows, heads, nope + dr] bf16, w_uk [heads, nope, dc] bf16 -> [rows, heads, dc + dr]: absorbed latent query
    with the rotated rotary part appended."""
    rows, heads, dq = q.shape
    if out is None:
        out = torch.empty(rows, heads, dc + dr, dtype=torch.bfloat16, device=q.device)
    call("dgpp_mla_q_absorb", ptr(q), ptr(w_uk), ptr(inv_freq), ptr(positions), ptr(out), rows, heads, dq - dr, dc, dr,
         stream_ptr())
    return out


def mla_v_up(lat, w_uv, out=None):
    """lat [rows, heads, dc] bf16, w_uv [heads, v, dc] bf16 -> [rows, heads * v] bf16."""
    rows, heads, dc = lat.shape
    v = w_uv.shape[1]
    if out is None:
        out = torch.empty(rows, heads * v, dtype=torch.bfloat16, device=lat.device)
    call("dgpp_mla_v_up", ptr(lat), ptr(w_uv), ptr(out), rows, heads, v, dc, stream_ptr())
    return out


_lib.declare("dgpp_dsa_index_tc", [P, P, P, P, P, P, P, I, I, I, I, I, I, I, P])


_lib.declare("dgpp_dsa_index_tc_fp8", [P, P, P, P, P, P, P, P, I, I, I, I, I, I, I, P])
_lib.declare("dgpp_dsa_key_append_fp8", [P, L, P, P, P, I, I, P, P, I, P])


def dsa_key_append_fp8(k_rows, positions, row_req, block_table, cache, kscale) -> None:
    """Index keys [rows, 128] bf16 of new tokens -> e4m3 bytes in the paged cache [blocks, page, 128] uint8 with one fp32
    scale per token in kscale [blocks, page] (amax / 448)."""
    _chk(k_rows, torch.bfloat16, "k_rows")
    assert cache.dtype == torch.uint8 and k_rows.shape[1] == 128 and cache.shape[2] == 128
    call("dgpp_dsa_key_append_fp8", ptr(k_rows), k_rows.stride(0), ptr(positions), ptr(row_req), ptr(block_table),
         block_table.shape[1], cache.shape[1], ptr(cache), ptr(kscale), k_rows.shape[0], stream_ptr())


def dsa_index(q_idx, w_idx, k_idx, block_table, row_req, positions, max_ctx: int, scores=None,
              tensor_cores: Optional[bool] = None, k_scale=None):
    """Lightning-indexer scores [rows, max_ctx] fp32 (-inf beyond each row's position).
    q_idx: [rows, hi, di] bf16, w_idx: [rows, hi] fp32, k_idx: paged [blocks, page, di] bf16, or e4m3 bytes (uint8) with
    k_scale [blocks, page] fp32 per-token scales (tensor-core kernel only, two-term e4m3 queries).
    Index dims of 128 with up to 64 heads run on the tensor cores (tensor_cores=False: the CUDA-core kernel)."""
    rows, hi, di = q_idx.shape
    if scores is None:
        scores = torch.empty(rows, max_ctx, dtype=torch.float32, device=q_idx.device)
    if k_idx.dtype == torch.uint8:
        assert k_scale is not None and di == 128 and hi <= 64 and k_idx.shape[1] in (16, 32, 64, 128)
        call("dgpp_dsa_index_tc_fp8", ptr(q_idx), ptr(w_idx), ptr(k_idx), ptr(k_scale), ptr(block_table), ptr(row_req),
             ptr(positions), ptr(scores), rows, hi, di, k_idx.shape[1], block_table.shape[1], k_idx.shape[0], scores.shape[1],
             stream_ptr())
        return scores
    if tensor_cores is None:
        tensor_cores = di == 128 and hi <= 64 and k_idx.shape[1] in (16, 32, 64, 128)
    if tensor_cores:
        call("dgpp_dsa_index_tc", ptr(q_idx), ptr(w_idx), ptr(k_idx), ptr(block_table), ptr(row_req), ptr(positions),
             ptr(scores), rows, hi, di, k_idx.shape[1], block_table.shape[1], k_idx.shape[0], scores.shape[1], stream_ptr())
        return scores
    call("dgpp_dsa_index", ptr(q_idx), ptr(w_idx), ptr(k_idx), ptr(block_table), ptr(row_req), ptr(positions),
         ptr(scores), rows, hi, di, k_idx.shape[1], block_table.shape[1], scores.shape[1], stream_ptr())
    return scores


def topk_select(scores, positions, k: int, out=None):
    """Exact top-k token positions per row among positions 0..positions[row] (ties to the lower position),
    ascending, -1 padded."""
    rows = scores.shape[0]
    if out is None:
        out = torch.empty(rows, k, dtype=torch.int32, device=scores.device)
    call("dgpp_topk_select", ptr(scores), scores.stride(0), ptr(positions), ptr(out), rows, k, stream_ptr())
    return out


# ---------------------------------------------------------------------------------------------- low-rank adapters
_lib.declare("dgpp_lora_apply", [P, L, P, P, P, P, L, F, I, I, I, I, P])


def lora_apply(x, a, b, out, scale: float, scratch=None):
    """out += scale * (x @ a.T) @ b.T in place.  x [T, K] bf16, a [r, K] bf16, b [N, r] bf16, out [T, N] bf16;
    the rank-r intermediate stays in fp32 (`scratch`: >= T * r floats)."""
    _chk(x, torch.bfloat16, "x")
    _chk(out, torch.bfloat16, "out")
    rows, k = x.shape
    r, n = a.shape[0], b.shape[0]
    assert a.shape == (r, k) and b.shape == (n, r) and out.shape == (rows, n) and a.is_contiguous() and b.is_contiguous()
    if scratch is None:
        scratch = torch.empty(rows * r, dtype=torch.float32, device=x.device)
    assert scratch.numel() >= rows * r
    call("dgpp_lora_apply", ptr(x), x.stride(0), ptr(a), ptr(b), ptr(scratch), ptr(out), out.stride(0), float(scale),
         rows, n, k, r, stream_ptr())
    return out
