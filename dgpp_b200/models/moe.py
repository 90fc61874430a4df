"""Mixture-of-experts feed-forward block: sigmoid (or softmax) router with selection bias and group-limited top-k,
routed SwiGLU experts with NVFP4 weights stacked into one matrix, optional shared experts, ordered accumulation.

* ``moe_reference``  PyTorch oracle of the numerics contract (fp32 router, weights from uncorrected scores, ids
  ascending = accumulation order, bf16 rounding points of the expert MLP).
* ``MoEBlock.forward`` the sm_100a path for decode-sized batches (rows <= token tile): router kernel, active-expert
  list, ONE grouped block-scaled GEMM launch for every active expert's gate/up, fused SwiGLU + quantiser over the
  slots, ONE grouped GEMM for the down projections, ordered combine.  Every token is a column of every active
  expert's MMA (the MMA N minimum is 16 anyway); the combine picks each token's experts.  Larger batches fall back
  to per-expert GEMMs over gathered rows.
(numerics: src/kernels/glm_moe.cu:86-331,1447 and the reference tree's own design notes (lines 1293-1413 of its top-level design document).)
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional

import torch

from ..ops import core as ops
from ..ops import reference as ref
from ..quant.formats import QuantLinear, tile_scales
from .dense import quantize_like_random

BF = torch.bfloat16


@dataclass
class MoEConfig:
    hidden: int = 2048
    experts: int = 64
    top_k: int = 8
    moe_ffn: int = 1024
    shared_ffn: int = 0            # 0: no shared expert
    n_group: int = 1
    topk_group: int = 1
    router: str = "sigmoid"        # or "softmax"
    norm_topk_prob: bool = True
    routed_scaling: float = 1.0
    swiglu_limit: float = 0.0
    swiglu_alpha: float = 0.0      # > 0: gate * sigmoid(alpha * gate) * (up + 1) instead of silu(gate) * up


@dataclass
class MoEWeights:
    cfg: MoEConfig
    gate: torch.Tensor                     # [E, H] bf16
    bias: Optional[torch.Tensor]           # [E] fp32 selection correction
    experts_gu: List[QuantLinear]          # per expert [2I, H]
    experts_down: List[QuantLinear]        # per expert [H, I]
    shared_gu: Optional[QuantLinear] = None
    shared_down: Optional[QuantLinear] = None
    # stacked device views for the grouped GEMM (built by `stack`)
    shared_gu_k: Optional[QuantLinear] = None
    shared_down_k: Optional[QuantLinear] = None
    gu_q: Optional[torch.Tensor] = None
    gu_sf: Optional[torch.Tensor] = None
    gu_alpha: Optional[torch.Tensor] = None
    down_q: Optional[torch.Tensor] = None
    down_sf: Optional[torch.Tensor] = None
    down_alpha: Optional[torch.Tensor] = None
    # expert parallelism: this rank holds experts [e_begin, e_end) (experts_gu / experts_down are that slice); the
    # router weights are replicated; the shared expert lives on rank 0
    e_begin: int = 0
    e_end: int = 0
    # False: `stack` drops the per-expert tensors once the stacked device tensors exist (large models: the lists would
    # double the expert memory; only the PyTorch oracles and the expert-loop check read them)
    KEEP_EXPERT_LISTS = True

    @staticmethod
    def random_init(cfg: MoEConfig, device, seed: int = 0, std: float = 0.02, fmt: str = "nvfp4", ep_rank: int = 0,
                    ep_size: int = 1, shared_everywhere: bool = False) -> "MoEWeights":
        """Every rank draws all experts from the same seed and keeps its contiguous block, so the union over ranks
        is the model a single rank would build.  The shared expert lives on rank 0 when every rank sees every token
        (its output is summed once), on every rank when the tokens are sharded (shared_everywhere)."""
        from ..runtime import rt

        g = torch.Generator(device=device)
        g.manual_seed(seed)
        rnd = lambda n, k: torch.randn(n, k, device=device, dtype=torch.float32, generator=g) * std
        gate = (rnd(cfg.experts, cfg.hidden) * 4).to(BF)
        bias = torch.randn(cfg.experts, device=device, generator=g) * 0.05
        e0, e1 = rt.expert_slice(cfg.experts, ep_size, ep_rank)
        gu, dn = [], []
        for e in range(cfg.experts):
            a, b = rnd(2 * cfg.moe_ffn, cfg.hidden), rnd(cfg.hidden, cfg.moe_ffn)
            if e0 <= e < e1:
                gu.append(quantize_like_random(a, fmt, std))
                dn.append(quantize_like_random(b, fmt, std))
        sgu = sdn = None
        if cfg.shared_ffn:
            a, b = rnd(2 * cfg.shared_ffn, cfg.hidden), rnd(cfg.hidden, cfg.shared_ffn)
            if ep_rank == 0 or shared_everywhere:
                sgu, sdn = quantize_like_random(a, fmt, std), quantize_like_random(b, fmt, std)
        w = MoEWeights(cfg, gate, bias, gu, dn, sgu, sdn, e_begin=e0, e_end=e1)
        if fmt in ("nvfp4", "mxfp4") and torch.device(device).type == "cuda":
            w.stack()
        return w

    def stack(self) -> None:
        """Concatenate the experts' payloads / tiled scales along N: one tensor map serves every expert."""
        def cat(ws: List[QuantLinear]):
            if ws and ws[0].fmt == "mxfp4":
                # MXFP4 experts stream through the same grouped block-scaled GEMM: the e2m1 bytes stay as stored, the
                # power-of-two block scales are re-expressed exactly as e4m3 per 16 + an fp32 tensor scale
                from ..quant.formats import mxfp4_as_nvfp4
                conv = [mxfp4_as_nvfp4(w) for w in ws]
                if any(c is None for c in conv):
                    return None, None, None
                ws = conv
            q = torch.cat([w.payload for w in ws]).contiguous()
            sf = torch.cat([tile_scales(w.scale.view(w.n, w.k // 16)).reshape(-1) for w in ws]).contiguous()
            al = torch.tensor([w.alpha for w in ws], dtype=torch.float32, device=q.device)
            return q, sf, al
        # A shared expert of the routed experts' shape rides in the same stack as one more expert (index = number of
        # local experts): the decode path then runs it inside the two grouped GEMMs as an always-listed slot instead of
        # two further launches and a quantiser of its own.
        self.shared_stacked = (self.shared_gu is not None and self.cfg.shared_ffn == self.cfg.moe_ffn
                               and bool(self.experts_gu) and self.shared_gu.fmt == self.experts_gu[0].fmt)
        extra_gu = [self.shared_gu] if self.shared_stacked else []
        extra_dn = [self.shared_down] if self.shared_stacked else []
        self.gu_q, self.gu_sf, self.gu_alpha = cat(self.experts_gu + extra_gu)
        if self.gu_q is not None and not MoEWeights.KEEP_EXPERT_LISTS:
            self.experts_gu = []                    # (the per-expert tensors only serve the oracles)
        self.down_q, self.down_sf, self.down_alpha = cat(self.experts_down + extra_dn)
        if self.down_q is not None and not MoEWeights.KEEP_EXPERT_LISTS:
            self.experts_down = []
        if self.gu_q is None or self.down_q is None:
            self.gu_q = self.down_q = None          # a scale range too wide to re-express: the oracle path serves it
        # kernel views of the shared expert (the stored MXFP4 tensors stay the oracle's)
        self.shared_gu_k, self.shared_down_k = self.shared_gu, self.shared_down
        if self.shared_gu is not None and self.shared_gu.fmt == "mxfp4":
            from ..quant.formats import mxfp4_as_nvfp4
            self.shared_gu_k, self.shared_down_k = mxfp4_as_nvfp4(self.shared_gu), mxfp4_as_nvfp4(self.shared_down)
            if self.shared_gu_k is None or self.shared_down_k is None:
                self.gu_q = self.down_q = None


def route_reference(x: torch.Tensor, w: MoEWeights):
    """fp32 router of the contract.  Returns (ids [T, k] ascending, weights [T, k] fp32, logits [T, E])."""
    c = w.cfg
    logits = x.float() @ w.gate.float().t()
    scores = torch.softmax(logits, -1) if c.router == "softmax" else torch.sigmoid(logits)
    sel = scores + (w.bias.float() if w.bias is not None else 0.0)
    if c.n_group > 1:
        T = x.shape[0]
        per = c.experts // c.n_group
        gs = sel.view(T, c.n_group, per)
        top2 = gs.topk(min(2, per), dim=-1).values.sum(-1)                # [T, n_group]
        keep = torch.zeros_like(top2, dtype=torch.bool)
        order = torch.argsort(-top2, dim=-1, stable=True)[:, :c.topk_group]   # ties -> lower group id
        keep.scatter_(1, order, True)
        sel = torch.where(keep.unsqueeze(-1).expand(T, c.n_group, per).reshape(T, c.experts), sel,
                          torch.full_like(sel, float("-inf")))
    order = torch.argsort(-sel, dim=-1, stable=True)[:, :c.top_k]         # ties -> lower expert id
    ids = torch.sort(order, dim=-1).values
    wts = scores.gather(1, ids)
    if c.norm_topk_prob:
        wts = wts / (wts.sum(-1, keepdim=True) + 1e-20)
    return ids.to(torch.int32), wts * c.routed_scaling, logits


def moe_reference(x: torch.Tensor, w: MoEWeights, ids=None, wts=None) -> torch.Tensor:
    """x [T, H] (normed hidden, bf16).  Expert MLP: bf16(bf16(silu(g)) * u) -> down; fp32 ordered accumulation of
    w_e * y_e over ascending expert ids, shared expert added last, one bf16 rounding."""
    c = w.cfg
    if ids is None:
        ids, wts, _ = route_reference(x, w)
    T = x.shape[0]
    acc = torch.zeros(T, c.hidden, dtype=torch.float32, device=x.device)
    e0, e1 = w.e_begin, (w.e_end or c.experts)
    for e in sorted(set(ids.flatten().tolist())):
        if not (e0 <= e < e1):
            continue                      # another rank's expert
        rows = (ids == e).any(-1).nonzero().flatten()
        xe = x[rows]
        h = ref.linear(xe, w.experts_gu[e - e0])
        y = ref.linear(ref.swiglu(h, c.swiglu_limit, c.swiglu_alpha), w.experts_down[e - e0])
        we = (wts * (ids == e)).sum(-1)[rows]
        acc[rows] += we.unsqueeze(-1) * y.float()
    if w.shared_gu is not None:
        acc += ref.linear(ref.swiglu(ref.linear(x, w.shared_gu), c.swiglu_limit, c.swiglu_alpha), w.shared_down).float()
    return ref.act(acc)


class MoEBlock:
    """Device buffers + launch sequence of one MoE block for up to `max_rows` decode rows."""

    # residual NVFP4 terms of the activations at prefill sizes (tiles of 64 rows).  3 = the decode path's arithmetic
    # (near-bf16 activations); 1 = plain W4A4 (4-bit activations, a third of the tensor-core and quantiser work).
    # Class-wide so one deployment key sets it for every block.
    PREFILL_TERMS = 3

    def __init__(self, w: MoEWeights, max_rows: int, device, act_terms: int = 3, prefill_terms: Optional[int] = None,
                 pool: Optional[dict] = None):
        """pool: a dict shared by the blocks of one runner (same shapes, one block running at a time): the expert
        output and quantiser buffers are then allocated once instead of once per layer.  The routing tables
        (`ids`, `wts`, the active list) stay per block."""
        c = w.cfg
        assert w.gu_q is not None, "call MoEWeights.stack() on the device first"
        self.w, self.c, self.dev, self.terms = w, c, device, act_terms
        self.prefill_terms = prefill_terms or self.PREFILL_TERMS
        self.bn = 16 if max_rows <= 16 else (32 if max_rows <= 32 else 64)
        assert max_rows <= self.bn and act_terms * self.bn <= 256
        self.max_rows = max_rows
        self.e0, self.e1 = w.e_begin, (w.e_end or c.experts)
        self.local_experts = self.e1 - self.e0
        self.slots = min(self.local_experts, max_rows * c.top_k)
        i32 = dict(dtype=torch.int32, device=device)
        self.ids = torch.zeros(max_rows, c.top_k, **i32)
        self.wts = torch.zeros(max_rows, c.top_k, dtype=torch.float32, device=device)
        # with a stacked shared expert the slot after the routed ones always lists it
        self.sh_slot = self.slots if getattr(w, "shared_stacked", False) else -1
        nslots = self.slots + (1 if self.sh_slot >= 0 else 0)
        self.stack_experts = self.local_experts + (1 if self.sh_slot >= 0 else 0)
        self.group_list = torch.full((nslots,), -1, **i32)
        if self.sh_slot >= 0:
            self.group_list[self.sh_slot] = self.local_experts
        self.slot_of = torch.full((c.experts,), -1, **i32)
        self.n_active = torch.zeros(1, **i32)

        def shared(name, make):
            if pool is None:
                return make()
            key = (name, nslots, self.bn, max_rows, c.hidden, c.moe_ffn, c.shared_ffn, act_terms)
            if key not in pool:
                pool[key] = make()
            return pool[key]

        self.h = shared("h", lambda: torch.zeros(nslots, self.bn, 2 * c.moe_ffn, dtype=BF, device=device))
        self.y = shared("y", lambda: torch.zeros(nslots, self.bn, c.hidden, dtype=BF, device=device))
        self.qa_in = shared("qa_in", lambda: ops.QuantAct(self.bn, c.hidden, act_terms, self.bn, device))
        self.qa_mid = shared("qa_mid", lambda: ops.QuantAct(nslots * self.bn, c.moe_ffn, act_terms, self.bn, device))
        self.nslots = nslots
        self.shared = None
        if w.shared_gu is not None and self.sh_slot < 0:
            self.shared = shared("shared", lambda: torch.zeros(max_rows, c.hidden, dtype=BF, device=device))
            self.sh_gu = shared("sh_gu", lambda: torch.zeros(max_rows, 2 * c.shared_ffn, dtype=BF, device=device))
            self.qa_sh = shared("qa_sh", lambda: ops.QuantAct(self.bn, c.shared_ffn, act_terms, self.bn, device))

    def forward(self, xn: torch.Tensor, out: Optional[torch.Tensor], xa: Optional[ops.QuantAct] = None,
                push_comm=None) -> Optional[torch.Tensor]:
        """xn: [rows, H] bf16 normed hidden; xa: its NVFP4 terms when the caller's norm kernel already produced
        them.  out: [rows, H] bf16.  push_comm (expert parallelism): native peer communicator; this rank's partial
        sum over ITS experts is then pushed to every rank instead of being written to `out` (the next layer's
        fold + add + RMSNorm + quantise kernel sums the ranks)."""
        c, w = self.c, self.w
        rows = xn.shape[0]
        assert rows <= self.max_rows
        if xa is None:
            xa = ops.act_quant_nvfp4(xn, self.terms, out=self.qa_in)
        ops.moe_route(xn, w.gate, w.bias, c.top_k, c.n_group, c.topk_group, c.router == "softmax", c.norm_topk_prob,
                      c.routed_scaling, ids=self.ids[:rows], weights=self.wts[:rows])
        ops.moe_active(self.ids[:rows], rows, c.experts, self.slots, self.group_list, self.slot_of, self.n_active,
                       self.e0, self.e1)
        ops.gemm_fp4_grouped(xa, w.gu_q, w.gu_sf, w.gu_alpha, self.h, rows, 2 * c.moe_ffn, c.hidden, self.stack_experts,
                             self.group_list, group_b=False)
        xm = ops.act_quant_nvfp4(self.h.view(self.nslots * self.bn, 2 * c.moe_ffn), self.terms, out=self.qa_mid,
                                 mode="swiglu", limit=c.swiglu_limit, alpha=c.swiglu_alpha, group_list=self.group_list, group_rows=rows)
        ops.gemm_fp4_grouped(xm, w.down_q, w.down_sf, w.down_alpha, self.y, rows, c.hidden, c.moe_ffn, self.stack_experts,
                             self.group_list, group_b=True)
        sh = self.y[self.sh_slot] if self.sh_slot >= 0 else None          # [bn, H]: the shared expert's rows
        if self.shared is not None:
            ops.gemm_fp4(xa, w.shared_gu_k, out=self.sh_gu[:rows])
            xs = ops.act_quant_nvfp4(self.sh_gu[:rows], self.terms, out=self.qa_sh, mode="swiglu", limit=c.swiglu_limit, alpha=c.swiglu_alpha)
            ops.gemm_fp4(xs, w.shared_down_k, out=self.shared[:rows])
            sh = self.shared
        if push_comm:
            ops.moe_combine_push(self.y, sh, self.ids[:rows], self.wts[:rows], self.slot_of, push_comm, rows)
            return None
        return ops.moe_combine(self.y, sh, self.ids[:rows], self.wts[:rows], self.slot_of, out, rows)

    def forward_gathered(self, xn: torch.Tensor) -> torch.Tensor:
        """Prefill-sized batches, all on the device: router, counting sort of the (token, k) pairs by expert into tiles
        of 64 rows, row gather, then the decode path's kernels with every tile as one slot -- residual-term quantiser,
        grouped block-scaled gate/up GEMM, SwiGLU quantiser, grouped down GEMM -- and the ordered combine.  The tile
        buffers are shared by all blocks of a device (one MoE block runs at a time).
        (reference counterparts: src/kernels/glm_moe.cu:1382 segment count, :1553 tile list, :1121 grouped MMA.)"""
        c, w = self.c, self.w
        T = xn.shape[0]
        bn, R = 64, self.prefill_terms
        max_tiles = (T * c.top_k + bn - 1) // bn + self.local_experts
        ws = _prefill_workspace(xn.device, max_tiles, bn, c.hidden, c.moe_ffn, R)
        ids, wts = ops.moe_route(xn, w.gate, w.bias, c.top_k, c.n_group, c.topk_group, c.router == "softmax",
                                 c.norm_topk_prob, c.routed_scaling)
        tiles = ws["tile_expert"][:max_tiles]
        pair_row, _, _ = ops.moe_segment_sort(ids, bn, max_tiles, self.e0, self.e1, ws["pair_row"][:T * c.top_k], tiles,
                                              ws["n_tiles"])
        rows = max_tiles * bn
        xs, h, y = ws["xs"][:rows], ws["h"][:max_tiles], ws["y"][:max_tiles]
        ops.moe_gather_rows(xn, pair_row, xs, c.top_k)
        xa = ops.act_quant_nvfp4(xs, R, out=ws["qa_x"], group_list=tiles, group_rows=bn)
        ops.gemm_fp4_grouped(xa, w.gu_q, w.gu_sf, w.gu_alpha, h, bn, 2 * c.moe_ffn, c.hidden, self.local_experts, tiles,
                             group_b=True)
        xm = ops.act_quant_nvfp4(h.view(rows, 2 * c.moe_ffn), R, out=ws["qa_mid"], mode="swiglu", limit=c.swiglu_limit, alpha=c.swiglu_alpha,
                                 group_list=tiles, group_rows=bn)
        ops.gemm_fp4_grouped(xm, w.down_q, w.down_sf, w.down_alpha, y, bn, c.hidden, c.moe_ffn, self.local_experts, tiles,
                             group_b=True)
        sh = None
        if w.shared_gu is not None:
            sh = ops.linear(ops.swiglu(ops.linear(xn, w.shared_gu), limit=c.swiglu_limit, alpha=c.swiglu_alpha), w.shared_down)
        out = torch.empty(T, c.hidden, dtype=BF, device=xn.device)
        return ops.moe_combine_rows(y.view(rows, c.hidden), sh, pair_row, wts, out)

    def forward_looped(self, xn: torch.Tensor) -> torch.Tensor:
        """Oracle of forward_gathered: one exact W4A16 GEMM pair per active expert over its gathered rows (host loop)."""
        c, w = self.c, self.w
        ids, wts = ops.moe_route(xn, w.gate, w.bias, c.top_k, c.n_group, c.topk_group, c.router == "softmax",
                                 c.norm_topk_prob, c.routed_scaling)
        acc = torch.zeros(xn.shape[0], c.hidden, dtype=torch.float32, device=xn.device)
        for e in torch.unique(ids).tolist():
            if not (self.e0 <= e < self.e1):
                continue
            hit = ids == e
            rows = hit.any(-1).nonzero().flatten()
            xe = xn.index_select(0, rows).contiguous()
            h = ops.linear(xe, w.experts_gu[e - self.e0])
            y = ops.linear(ops.swiglu(h, limit=c.swiglu_limit, alpha=c.swiglu_alpha), w.experts_down[e - self.e0])
            acc.index_add_(0, rows, (wts * hit).sum(-1)[rows].unsqueeze(-1) * y.float())
        if w.shared_gu is not None:
            acc += ops.linear(ops.swiglu(ops.linear(xn, w.shared_gu), limit=c.swiglu_limit, alpha=c.swiglu_alpha), w.shared_down).float()
        return acc.to(BF)


_PREFILL_WS: dict = {}


def _prefill_workspace(device, max_tiles: int, bn: int, hidden: int, ffn: int, terms: int) -> dict:
    """Tile buffers of MoEBlock.forward_gathered, kept per (device, geometry) and grown to the largest tile count."""
    key = (str(device), bn, hidden, ffn, terms)
    ws = _PREFILL_WS.get(key)
    if ws is None or ws["max_tiles"] < max_tiles:
        rows = max_tiles * bn
        i32 = dict(dtype=torch.int32, device=device)
        ws = dict(max_tiles=max_tiles,
                  pair_row=torch.empty(rows, **i32), tile_expert=torch.full((max_tiles,), -1, **i32),
                  n_tiles=torch.zeros(1, **i32),
                  xs=torch.zeros(rows, hidden, dtype=BF, device=device),
                  h=torch.zeros(max_tiles, bn, 2 * ffn, dtype=BF, device=device),
                  y=torch.zeros(max_tiles, bn, hidden, dtype=BF, device=device),
                  qa_x=ops.QuantAct(rows, hidden, terms, bn, device),
                  qa_mid=ops.QuantAct(rows, ffn, terms, bn, device))
        _PREFILL_WS[key] = ws
    return ws
