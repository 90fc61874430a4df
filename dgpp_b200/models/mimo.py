"""Sliding-window / global hybrid GQA + mixture-of-experts family with a draft layer (MiMo-V2 style).

Layers interleave sliding-window attention (window W, one learned sink logit per head: a value-less softmax column,
own kv-head count and rotary base) with global attention on a per-layer pattern; q / k rotate on their first
`rotary_dim` dims; values are scaled by a constant before they enter the cache.  The first layers carry a dense SwiGLU
MLP, the others a sigmoid-routed MoE without a shared expert (selection bias on the key, picked scores normalised).
A draft (multi-token-prediction) layer, a sliding-window block with a dense MLP, reads
    proj([rmsnorm(hidden of position p) ; rmsnorm(embed(token p + 1))])
and predicts token p + 2 through the model's head; it keeps its own KV history per request, filled for every position
whose next token is known (`draft_append`), so that `draft` at the newest position sees the window it needs.

Oracle: ``MimoModel.forward_reference`` / ``draft_reference``; kernels: `rope_kv_write`, the paged decode attention
with window + sink (sliding layers, prefill rows included), tcgen05 attention (global layers), the MoE block, `rmsnorm`,
tensor-core linears.
(reference counterparts: src/models/mimo/forward.cpp, layers.cpp, attn_reference.cpp, kv_pool.cpp,
 src/kernels/sink_attn_impl.cuh.  The release's 192-wide q / k heads over 128-wide values need a padded head here and
 are not part of this build: one head width serves q, k and v.)
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import List, Optional

import torch

from ..ops import core as ops
from ..ops import reference as ref
from ..quant.formats import QuantLinear, quantize
from .moe import MoEBlock, MoEConfig, MoEWeights, moe_reference
from .rows import RowRunner

BF = torch.bfloat16


@dataclass
class MimoConfig:
    layers: int = 4
    hidden: int = 512
    q_heads: int = 8
    kv_heads: int = 2               # global layers
    swa_kv_heads: int = 4           # sliding-window layers
    head_dim: int = 128
    rotary_dim: int = 64
    rope_theta: float = 1e7         # global layers
    swa_rope_theta: float = 1e4     # sliding-window layers and the draft layer
    window: int = 32
    swa_layers: List[bool] = field(default_factory=list)     # empty: every layer but each 4th is sliding
    swa_sink: bool = True
    value_scale: float = 0.707
    dense_layers: int = 1           # the first layers carry the dense MLP
    ffn: int = 1024
    moe: Optional[MoEConfig] = None
    draft: bool = True
    eps: float = 1e-6
    vocab: int = 2048
    page: int = 64

    def is_swa(self, i: int) -> bool:
        return self.swa_layers[i] if self.swa_layers else (i + 1) % 4 != 0

    def is_moe(self, i: int) -> bool:
        return self.moe is not None and i >= self.dense_layers


@dataclass
class MimoLayer:
    swa: bool
    in_norm: torch.Tensor
    post_norm: torch.Tensor
    qkv: QuantLinear                 # [(hq + 2 hkv) d, H], hkv by the layer's kind; the value rows carry value_scale
    o: QuantLinear
    sink: Optional[torch.Tensor] = None      # [hq] fp32
    gate_up: Optional[QuantLinear] = None
    down: Optional[QuantLinear] = None
    moe: Optional[MoEWeights] = None


class MimoModel:
    def __init__(self, cfg: MimoConfig, embed, layers: List[MimoLayer], final_norm, head: QuantLinear, inv_ga, inv_swa):
        self.cfg, self.embed, self.layers, self.final_norm, self.head = cfg, embed, layers, final_norm, head
        self.inv_ga, self.inv_swa = inv_ga, inv_swa
        self.draft_proj: Optional[QuantLinear] = None         # [H, 2 H]
        self.draft_norm_h = self.draft_norm_e = self.draft_final_norm = None
        self.draft_layer: Optional[MimoLayer] = None

    def kv_heads_of(self, L: MimoLayer) -> int:
        return self.cfg.swa_kv_heads if L.swa else self.cfg.kv_heads

    @staticmethod
    def random_init(cfg: MimoConfig, device, seed: int = 0, std: float = 0.05, fmt: str = "bf16") -> "MimoModel":
        g = torch.Generator(device=device)
        g.manual_seed(seed)
        c, H, d = cfg, cfg.hidden, cfg.head_dim
        rnd = lambda *s: torch.randn(*s, device=device, dtype=torch.float32, generator=g)
        lin = lambda n, k: quantize(rnd(n, k) * std, fmt if (k % 256 == 0 or fmt == "bf16") else "bf16")
        nw = lambda n: (1 + 0.1 * rnd(n)).to(BF)

        def block(swa: bool, moe: bool, i: int) -> MimoLayer:
            hkv = c.swa_kv_heads if swa else c.kv_heads
            w = rnd((c.q_heads + 2 * hkv) * d, H) * std
            w[(c.q_heads + hkv) * d:] *= c.value_scale              # values enter the cache scaled
            L = MimoLayer(swa, nw(H), nw(H), quantize(w, fmt if fmt == "bf16" or H % 256 == 0 else "bf16"), lin(H, c.q_heads * d))
            if swa and c.swa_sink:
                L.sink = rnd(c.q_heads)
            if moe:
                L.moe = MoEWeights.random_init(c.moe, device, seed=seed * 1000 + i, std=std)
            else:
                L.gate_up, L.down = lin(2 * c.ffn, H), lin(H, c.ffn)
            return L

        layers = [block(c.is_swa(i), c.is_moe(i), i) for i in range(c.layers)]
        inv_ga, _ = ref.rope_inv_freq(c.rotary_dim, c.rope_theta, device)
        inv_swa, _ = ref.rope_inv_freq(c.rotary_dim, c.swa_rope_theta, device)
        m = MimoModel(cfg, (rnd(c.vocab, H) * std * 4).to(BF), layers, nw(H), quantize(rnd(c.vocab, H) * std, "bf16"),
                      inv_ga, inv_swa)
        if c.draft:
            m.draft_proj = quantize(rnd(H, 2 * H) * std, "bf16")
            m.draft_norm_h, m.draft_norm_e, m.draft_final_norm = nw(H), nw(H), nw(H)
            m.draft_layer = block(True, False, c.layers)
        return m

    # ------------------------------------------------------------------ oracle
    def _attention_reference(self, L: MimoLayer, xn: torch.Tensor, pos: torch.Tensor) -> torch.Tensor:
        c, d = self.cfg, self.cfg.head_dim
        T, hkv = xn.shape[0], self.kv_heads_of(L)
        nq, nkv = c.q_heads * d, hkv * d
        inv = self.inv_swa if L.swa else self.inv_ga
        qkv = ref.linear(xn, L.qkv).float()
        q = ref.apply_rope(qkv[:, :nq].view(T, c.q_heads, d), pos, inv, c.rotary_dim)
        k = ref.apply_rope(qkv[:, nq:nq + nkv].view(T, hkv, d), pos, inv, c.rotary_dim)
        v = ref._r(qkv[:, nq + nkv:].view(T, hkv, d))
        kq, ks = ref.quant_kv_fp8(k)
        vq, vs = ref.quant_kv_fp8(v)
        k = kq.view(torch.float8_e4m3fn).float() * ks.unsqueeze(-1)
        v = vq.view(torch.float8_e4m3fn).float() * vs.unsqueeze(-1)
        a = ref.attention(q, k, v, 1.0 / math.sqrt(d), causal_offset=0, window=c.window if L.swa else 0, sink=L.sink)
        return ref.linear(ref.act(a.reshape(T, nq)), L.o)

    def _ffn_reference(self, L: MimoLayer, xn: torch.Tensor) -> torch.Tensor:
        if L.moe is not None:
            return moe_reference(xn, L.moe)
        return ref.linear(ref.swiglu(ref.linear(xn, L.gate_up)), L.down)

    def _block_reference(self, L: MimoLayer, R, delta, pos):
        c = self.cfg
        xn, R = ref.rmsnorm(R, L.in_norm, c.eps, delta=delta)
        delta = self._attention_reference(L, xn, pos)
        xn, R = ref.rmsnorm(R, L.post_norm, c.eps, delta=delta)
        return R, self._ffn_reference(L, xn)

    def forward_reference(self, tokens: torch.Tensor, return_hidden: bool = False):
        """fp32 logits [T, V] of one request from position 0 (and the bf16 final-norm input rows)."""
        c = self.cfg
        dev = self.embed.device
        pos = torch.arange(tokens.numel(), device=dev)
        R, delta = ref.embed_gather(tokens.to(dev), self.embed), None
        for L in self.layers:
            R, delta = self._block_reference(L, R, delta, pos)
        xn, hidden = ref.rmsnorm(R, self.final_norm, c.eps, delta=delta)
        logits = ref.linear(xn, self.head, out_fp32=True)
        return (logits, hidden) if return_hidden else logits

    def draft_reference(self, hidden: torch.Tensor, next_tokens: torch.Tensor) -> torch.Tensor:
        """hidden [T, H] (rows 0 .. T-1 of the main model, before its final norm), next_tokens [T] (tokens 1 .. T)
        -> fp32 draft logits [T, V]: row p predicts token p + 2."""
        c = self.cfg
        pos = torch.arange(hidden.shape[0], device=hidden.device)
        hn = ref.rmsnorm(hidden, self.draft_norm_h, c.eps)[0]
        en = ref.rmsnorm(ref.embed_gather(next_tokens.to(hidden.device), self.embed), self.draft_norm_e, c.eps)[0]
        R = ref.linear(torch.cat([hn, en], -1), self.draft_proj)
        R, delta = self._block_reference(self.draft_layer, R, None, pos)
        xn, _ = ref.rmsnorm(R, self.draft_final_norm, c.eps, delta=delta)
        return ref.linear(xn, self.head, out_fp32=True)


class _DualKV:
    """The global layers' cache (the attributes the row plumbing reads) with the sliding layers' and the draft layer's
    caches reserved and released alongside it."""

    def __init__(self, ga, others):
        self.ga, self.others = ga, others
        self.layers, self.block_table, self.page = ga.layers, ga.block_table, ga.page

    def reserve(self, slot: int, tokens: int) -> bool:
        return self.ga.reserve(slot, tokens) and all(o.reserve(slot, tokens) for o in self.others)

    def release(self, slot: int) -> None:
        self.ga.release(slot)
        for o in self.others:
            o.release(slot)


class MimoRunner(RowRunner):
    def __init__(self, model: MimoModel, max_rows: int, slots: int, max_seq_len: int, device):
        from ..engine.kv_cache import PagedKV

        c = model.cfg
        self.m, self.c = model, c
        self.ga_index = {i: j for j, i in enumerate(i for i, L in enumerate(model.layers) if not L.swa)}
        self.swa_index = {i: j for j, i in enumerate(i for i, L in enumerate(model.layers) if L.swa)}
        self._init_rows(slots, device, kv_layers=max(len(self.ga_index), 1), kv_heads=c.kv_heads, q_heads=c.q_heads,
                        head_dim=c.head_dim, page=c.page, max_seq_len=max_seq_len, max_rows=max_rows)
        ga = self.kv
        self.swa_kv = PagedKV(max(len(self.swa_index), 1), c.swa_kv_heads, c.head_dim, ga.num_blocks, slots, ga.max_blocks,
                              c.page, True, device)
        self.draft_kv = PagedKV(1, c.swa_kv_heads, c.head_dim, ga.num_blocks, slots, ga.max_blocks, c.page, True,
                                device) if model.draft_layer is not None else None
        self.kv = _DualKV(ga, [self.swa_kv] + ([self.draft_kv] if self.draft_kv is not None else []))
        pool = {}
        self.moe = {i: MoEBlock(L.moe, min(max_rows, 16), device, pool=pool) for i, L in enumerate(model.layers)
                    if L.moe is not None and L.moe.gu_q is not None}
        e = lambda *s: torch.empty(*s, dtype=BF, device=device)
        H, d = c.hidden, c.head_dim
        self.R, self.xn, self.y, self.hidden = e(max_rows, H), e(max_rows, H), e(max_rows, H), e(max_rows, H)
        self.qkv_ga = e(max_rows, (c.q_heads + 2 * c.kv_heads) * d)
        self.qkv_swa = e(max_rows, (c.q_heads + 2 * c.swa_kv_heads) * d)
        self.attn = e(max_rows, c.q_heads * d)
        self.gu, self.act = e(max_rows, 2 * c.ffn), e(max_rows, c.ffn)
        self.cat = e(max_rows, 2 * H)
        self.draft_len = [0] * slots          # the draft cache holds positions < draft_len

    def _reset_state(self, slot: int) -> None:
        self.draft_len[slot] = 0

    def _block(self, i: int, L: MimoLayer, cache, bt, R, delta, positions, row_req, chunk_slot, pos0):
        """One transformer block; returns the FFN output (the next block's delta)."""
        c, rows = self.c, R.shape[0]
        xn, y, attn = self.xn[:rows], self.y[:rows], self.attn[:rows]
        ops.rmsnorm(R, L.in_norm, c.eps, delta=delta, out=xn)
        if L.swa:
            qkv = ops.linear(xn, L.qkv, out=self.qkv_swa[:rows])
            ops.rope_kv_write(qkv, positions, row_req, bt, self.m.inv_swa, cache, c.q_heads, c.swa_kv_heads, c.head_dim,
                              rot_dim=c.rotary_dim)
            ops.attn_decode(qkv, qkv.stride(0), cache, bt, row_req, positions, c.q_heads, c.swa_kv_heads, c.head_dim,
                            self.att_scale, out=attn, window=c.window, sink=L.sink)
        else:
            qkv = ops.linear(xn, L.qkv, out=self.qkv_ga[:rows])
            # rotary table of the global layers; K / V append and attention on the shared row plumbing
            hq, hkv, d = self.att_q, self.att_kv, self.att_d
            ops.rope_kv_write(qkv, positions, row_req, bt, self.m.inv_ga, cache, hq, hkv, d, rot_dim=c.rotary_dim)
            if self.tc_attn and chunk_slot is not None and pos0 is not None:
                ops.attn_prefill_tc(qkv, qkv.stride(0), cache, bt[chunk_slot], pos0, hq, hkv, d, self.att_scale, out=attn,
                                    rows=rows)
            elif self.tc_attn and rows <= 32:
                splits = max(1, min(32, -(-160 // (hkv * rows))))
                ops.attn_decode_tc(qkv, qkv.stride(0), cache, bt, row_req, positions, hq, hkv, d, self.att_scale,
                                   splits=splits, scratch=self.att_scratch, out=attn)
            else:
                ops.attn_decode(qkv, qkv.stride(0), cache, bt, row_req, positions, hq, hkv, d, self.att_scale, out=attn)
        ops.linear(attn, L.o, out=y)
        ops.rmsnorm(R, L.post_norm, c.eps, delta=y, out=xn)
        if L.moe is None:
            gu = ops.linear(xn, L.gate_up, out=self.gu[:rows])
            ops.linear(ops.swiglu(gu, out=self.act[:rows]), L.down, out=y)
        else:
            blk = self.moe.get(i)
            if blk is not None and rows <= blk.max_rows:
                blk.forward(xn, y)
            elif blk is not None:
                y.copy_(blk.forward_gathered(xn))
            else:
                y.copy_(moe_reference(xn, L.moe))
        return y

    @torch.no_grad()
    def forward(self, tokens, positions, row_req, chunk_slot=None, all_logits=True, pos0=None, extra=None):
        m, c = self.m, self.c
        rows = tokens.shape[0]
        R = ops.embed_gather(tokens, m.embed, out=self.R[:rows])
        delta = None
        for i, L in enumerate(m.layers):
            if L.swa:
                cache, bt = self.swa_kv.layers[self.swa_index[i]], self.swa_kv.block_table
            else:
                cache, bt = self.kv.layers[self.ga_index[i]], self.kv.block_table
            delta = self._block(i, L, cache, bt, R, delta, positions, row_req, chunk_slot, pos0)
        xn = ops.rmsnorm(R, m.final_norm, c.eps, delta=delta, out=self.xn[:rows], resid_out=self.hidden[:rows])
        sel = xn if all_logits else xn[rows - 1:rows]
        return ops.gemm_tc(sel, m.head, out32=torch.empty(sel.shape[0], c.vocab, dtype=torch.float32, device=self.dev))

    # ------------------------------------------------------------------ draft layer
    @torch.no_grad()
    def draft_rows(self, slot: int, hidden: torch.Tensor, next_tokens: List[int]) -> torch.Tensor:
        """Feeds the draft layer the pairs (hidden of position p, token p + 1) for the consecutive positions
        p = draft_len .. draft_len + n - 1 of request `slot` (its KV history grows by n) and returns the fp32 draft
        logits [n, V]; the last row is the proposal for the token after the newest one."""
        m, c = self.m, self.c
        assert m.draft_layer is not None, "the model has no draft layer"
        n, p0 = hidden.shape[0], self.draft_len[slot]
        assert n == len(next_tokens) and n <= self.max_rows
        assert self.draft_kv.reserve(slot, p0 + n), "KV pool exhausted"
        pos = torch.arange(p0, p0 + n, dtype=torch.int32, device=self.dev)
        req = torch.full((n,), slot, dtype=torch.int32, device=self.dev)
        tok = torch.tensor(next_tokens, dtype=torch.int32, device=self.dev)
        cat = self.cat[:n]
        cat[:, :c.hidden].copy_(ops.rmsnorm(hidden, m.draft_norm_h, c.eps))
        cat[:, c.hidden:].copy_(ops.rmsnorm(ops.embed_gather(tok, m.embed), m.draft_norm_e, c.eps))
        R = ops.linear(cat, m.draft_proj, out=self.R[:n])
        delta = self._block(-1, m.draft_layer, self.draft_kv.layers[0], self.draft_kv.block_table, R, None, pos, req, None, None)
        xn = ops.rmsnorm(R, m.draft_final_norm, c.eps, delta=delta, out=self.xn[:n])
        self.draft_len[slot] = p0 + n
        return ops.gemm_tc(xn, m.head, out32=torch.empty(n, c.vocab, dtype=torch.float32, device=self.dev))
