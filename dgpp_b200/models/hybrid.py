"""Hybrid decoder family: Gated DeltaNet layers with a full-attention GQA layer every `full_every` layers, dense or
mixture-of-experts feed-forward blocks, and an optional multi-token-prediction (MTP) head for speculative decoding.

``HybridModel.forward_reference`` is the PyTorch oracle (whole sequences, no cache); ``HybridRunner`` executes the
same model with the sm_100a kernels: paged FP8 KV for the attention layers, per-slot recurrent state for the GDN
layers, grouped NVFP4 expert GEMMs for the MoE blocks.  Prefill chunks of one request and batches of single decode
tokens share one code path.
MTP: depth-1 head  h' = block( W_p [norm(h_t) ; norm(embed(x_{t+1}))] ),  logits = lm_head(norm(h')) predicts
x_{t+2}; its proposals are verified by the target model in one pass (`rt.spec_judge`).
(reference counterparts: src/models/qwen/model35.cpp run_rows:2066-2399, glm/mtp.cpp; the reference tree's own DESIGN.md:1934-2123.)
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import List, Optional

import torch

from ..ops import core as ops
from ..ops import reference as ref
from ..quant.formats import QuantLinear, quantize
from .gdn import GdnConfig, GdnLayer, GdnState, GdnWeights, gdn_reference
from .moe import MoEBlock, MoEConfig, MoEWeights, moe_reference

BF = torch.bfloat16


@dataclass
class HybridConfig:
    layers: int = 8
    hidden: int = 1024
    full_every: int = 4            # layers i with (i + 1) % full_every == 0 are full attention
    q_heads: int = 8
    kv_heads: int = 2
    head_dim: int = 128
    gdn_k_heads: int = 4
    gdn_v_heads: int = 8
    gdn_dk: int = 128
    gdn_dv: int = 128
    ffn: int = 2816                # dense FFN width (moe is None)
    moe: Optional[MoEConfig] = None
    vocab: int = 4096
    rope_theta: float = 1e6
    eps: float = 1e-6
    mtp: bool = False
    page: int = 64

    def is_full(self, i: int) -> bool:
        return (i + 1) % self.full_every == 0

    def gdn_cfg(self) -> GdnConfig:
        return GdnConfig(self.hidden, self.gdn_k_heads, self.gdn_v_heads, self.gdn_dk, self.gdn_dv, 4, self.eps)


@dataclass
class HybridLayer:
    in_norm: torch.Tensor
    post_norm: torch.Tensor
    gdn: Optional[GdnWeights] = None
    qkv: Optional[QuantLinear] = None
    o: Optional[QuantLinear] = None
    gate_up: Optional[QuantLinear] = None
    down: Optional[QuantLinear] = None
    moe: Optional[MoEWeights] = None


@dataclass
class HybridModel:
    cfg: HybridConfig
    embed: torch.Tensor
    layers: List[HybridLayer]
    final_norm: torch.Tensor
    head: QuantLinear
    inv_freq: torch.Tensor
    mtp_proj: Optional[QuantLinear] = None        # [hidden, 2 * hidden]
    mtp_norm_h: Optional[torch.Tensor] = None
    mtp_norm_e: Optional[torch.Tensor] = None
    mtp_layer: Optional[HybridLayer] = None       # one full-attention block

    @staticmethod
    def random_init(cfg: HybridConfig, device, seed: int = 0, std: float = 0.05, fmt: str = "bf16") -> "HybridModel":
        g = torch.Generator(device=device)
        g.manual_seed(seed)
        H, d = cfg.hidden, cfg.head_dim
        rnd = lambda n, k: torch.randn(n, k, device=device, dtype=torch.float32, generator=g) * std
        ones = lambda n: torch.ones(n, device=device, dtype=BF)

        def attn_block(i):
            L = HybridLayer(ones(H), ones(H))
            L.qkv = quantize(rnd((cfg.q_heads + 2 * cfg.kv_heads) * d, H), fmt)
            L.o = quantize(rnd(H, cfg.q_heads * d), fmt)
            return L

        def ffn(L, i):
            if cfg.moe is not None:
                mc = MoEConfig(**{**cfg.moe.__dict__, "hidden": H})
                L.moe = MoEWeights.random_init(mc, device, seed=seed * 1000 + i, std=std,
                                               fmt="nvfp4" if torch.device(device).type == "cuda" else "bf16")
            else:
                L.gate_up = quantize(rnd(2 * cfg.ffn, H), fmt)
                L.down = quantize(rnd(H, cfg.ffn), fmt)
            return L

        layers = []
        for i in range(cfg.layers):
            if cfg.is_full(i):
                L = attn_block(i)
            else:
                L = HybridLayer(ones(H), ones(H), gdn=GdnWeights.random_init(cfg.gdn_cfg(), device, seed=seed * 77 + i, std=std, fmt=fmt))
            layers.append(ffn(L, i))
        embed = (torch.randn(cfg.vocab, H, device=device, generator=g) * std).to(BF)
        inv, _ = ref.rope_inv_freq(d, cfg.rope_theta, device)
        m = HybridModel(cfg, embed, layers, ones(H), quantize(rnd(cfg.vocab, H), "bf16"), inv)
        if cfg.mtp:
            m.mtp_proj = quantize(rnd(H, 2 * H), fmt)
            m.mtp_norm_h, m.mtp_norm_e = ones(H), ones(H)
            m.mtp_layer = ffn(attn_block(cfg.layers), cfg.layers)
        return m

    # ------------------------------------------------------------------ PyTorch oracle
    def _attn_reference(self, L: HybridLayer, xn: torch.Tensor, start_pos: int = 0) -> torch.Tensor:
        c = self.cfg
        T, d = xn.shape[0], c.head_dim
        qkv = ref.linear(xn, L.qkv).float()
        nq, nkv = c.q_heads * d, c.kv_heads * d
        pos = torch.arange(start_pos, start_pos + T, device=xn.device)
        q = ref.apply_rope(qkv[:, :nq].view(T, c.q_heads, d), pos, self.inv_freq, d)
        k = ref.apply_rope(qkv[:, nq:nq + nkv].view(T, c.kv_heads, d), pos, self.inv_freq, d)
        v = ref._r(qkv[:, nq + nkv:].view(T, c.kv_heads, d))
        a = ref.attention(q, k, v, 1.0 / math.sqrt(d), causal_offset=0)
        return ref.linear(ref.act(a.reshape(T, nq)), L.o)

    def _ffn_reference(self, L: HybridLayer, xn: torch.Tensor) -> torch.Tensor:
        if L.moe is not None:
            return moe_reference(xn, L.moe)
        return ref.linear(ref.swiglu(ref.linear(xn, L.gate_up)), L.down)

    def forward_reference(self, tokens: torch.Tensor, return_hidden: bool = False):
        """tokens [T] of one sequence from position 0.  Returns fp32 logits [T, vocab] (and the final hidden)."""
        c = self.cfg
        x = ref.embed_gather(tokens, self.embed)
        delta = None
        for i, L in enumerate(self.layers):
            xn, x = ref.rmsnorm(x, L.in_norm, c.eps, delta)
            if L.gdn is not None:
                cs = torch.zeros(3, c.gdn_cfg().conv_channels, device=x.device)
                ss = torch.zeros(c.gdn_v_heads, c.gdn_dk, c.gdn_dv, device=x.device)
                delta = gdn_reference(xn, L.gdn, cs, ss)
            else:
                delta = self._attn_reference(L, xn)
            xn, x = ref.rmsnorm(x, L.post_norm, c.eps, delta)
            delta = self._ffn_reference(L, xn)
        xn, x = ref.rmsnorm(x, self.final_norm, c.eps, delta)
        logits = ref.linear(xn, self.head, out_fp32=True)
        return (logits, x) if return_hidden else logits

    def mtp_reference(self, hidden: torch.Tensor, next_tokens: torch.Tensor) -> torch.Tensor:
        """hidden [T, H]: the residual stream after the last layer at positions 0..T-1 (before the final norm);
        next_tokens [T]: x_{t+1}.  Returns fp32 logits [T, vocab] for x_{t+2}."""
        c = self.cfg
        hn, _ = ref.rmsnorm(hidden, self.mtp_norm_h, c.eps)
        en, _ = ref.rmsnorm(ref.embed_gather(next_tokens, self.embed), self.mtp_norm_e, c.eps)
        x = ref.linear(torch.cat([hn, en], -1), self.mtp_proj)
        L = self.mtp_layer
        xn, x = ref.rmsnorm(x, L.in_norm, c.eps)
        delta = self._attn_reference(L, xn)
        xn, x = ref.rmsnorm(x, L.post_norm, c.eps, delta)
        delta = self._ffn_reference(L, xn)
        xn, _ = ref.rmsnorm(x, self.final_norm, c.eps, delta)
        return ref.linear(xn, self.head, out_fp32=True)


class HybridRunner:
    """Kernel execution of a HybridModel: paged FP8 KV for the attention layers, recurrent state pools for GDN."""

    def __init__(self, model: HybridModel, max_rows: int, slots: int, max_seq_len: int, device):
        from ..engine.kv_cache import PagedKV

        c = model.cfg
        self.m, self.c, self.dev, self.max_rows = model, c, device, max_rows
        n_full = sum(1 for i in range(c.layers) if c.is_full(i))
        blocks_per = (max_seq_len + c.page - 1) // c.page + 1
        self.kv = PagedKV(max(n_full, 1), c.kv_heads, c.head_dim, slots * blocks_per + 2, slots, blocks_per, c.page, True, device)
        self.gdn_state = {i: GdnState(c.gdn_cfg(), slots, device) for i in range(c.layers) if not c.is_full(i)}
        self.gdn = {i: GdnLayer(model.layers[i].gdn, max_rows, device) for i in self.gdn_state}
        self.full_index = {i: j for j, i in enumerate(i for i in range(c.layers) if c.is_full(i))}
        self.moe = {i: MoEBlock(L.moe, min(max_rows, 16), device) for i, L in enumerate(model.layers)
                    if L.moe is not None and L.moe.gu_q is not None}
        e = lambda *s: torch.empty(*s, dtype=BF, device=device)
        H, d = c.hidden, c.head_dim
        self.x, self.xn, self.delta = e(max_rows, H), e(max_rows, H), e(max_rows, H)
        self.qkv = e(max_rows, (c.q_heads + 2 * c.kv_heads) * d)
        self.attn = e(max_rows, c.q_heads * d)
        self.logits = torch.empty(max_rows, c.vocab, dtype=torch.float32, device=device)
        self.lengths = [0] * slots
        self.scale = 1.0 / math.sqrt(d)
        self.use_graphs, self._graphs, self._static = True, {}, {}
        # tensor-core attention (FP8 cache as stored): head_dim 128 / 256, up to 8 query heads per kv head
        self.tc_attn = (torch.device(device).type == "cuda" and d in (128, 256)
                        and c.q_heads // c.kv_heads in (1, 2, 4, 8))
        self.max_splits = 32
        if self.tc_attn:
            r = min(max_rows, 16)
            self.att_scratch = (torch.empty(r * c.q_heads * self.max_splits * 2, dtype=torch.float32, device=device),
                                torch.empty(r * c.q_heads * self.max_splits * d, dtype=torch.float32, device=device))

    def _decode_splits(self, rows: int) -> int:
        """KV splits of a decode pass: enough CTAs (kv heads x rows x splits) to cover the SMs; fixed per batch width,
        so a captured pass stays valid at every context length (a split past the end writes an empty partial)."""
        if rows > 16:
            return 1
        return max(1, min(self.max_splits, -(-160 // (self.c.kv_heads * rows))))

    def _state_tensors(self):
        """Tensors a decode pass updates in place besides the KV cache (recurrent layers' state)."""
        return [t for st in self.gdn_state.values() for t in (st.conv, st.ssm)]

    def reset(self, slot: int) -> None:
        self.kv.release(slot)
        self.lengths[slot] = 0
        for st in self.gdn_state.values():
            st.reset(slot)

    def _ffn(self, i: int, L: HybridLayer, xn: torch.Tensor, out: torch.Tensor) -> None:
        if L.moe is not None:
            blk = self.moe.get(i)
            if blk is not None and xn.shape[0] <= blk.max_rows:
                blk.forward(xn, out)
            elif blk is not None:
                out.copy_(blk.forward_gathered(xn))
            else:
                out.copy_(moe_reference(xn, L.moe))
            return
        ops.linear(ops.swiglu(ops.linear(xn, L.gate_up)), L.down, out=out)

    @torch.no_grad()
    def forward(self, tokens: torch.Tensor, positions: torch.Tensor, row_req: torch.Tensor, chunk_slot: Optional[int] = None,
                all_logits: bool = True, pos0: Optional[int] = None) -> torch.Tensor:
        """tokens / positions / row_req: int32 [rows] on the device.  chunk_slot given: the rows are consecutive
        tokens of that request starting at position pos0 (prefill chunk); otherwise one decode token per row.
        Returns fp32 logits [rows, V]."""
        m, c = self.m, self.c
        rows = tokens.shape[0]
        x, xn, delta = self.x[:rows], self.xn[:rows], self.delta[:rows]
        ops.embed_gather(tokens, m.embed, out=x)
        have = False
        for i, L in enumerate(m.layers):
            ops.rmsnorm(x, L.in_norm, c.eps, delta=delta if have else None, out=xn)
            if L.gdn is not None:
                self.gdn[i].forward(xn, self.gdn_state[i], delta, slot=chunk_slot or 0,
                                    row_slot=None if chunk_slot is not None else row_req)
            else:
                cache = self.kv.layers[self.full_index[i]]
                qkv, attn = self.qkv[:rows], self.attn[:rows]
                ops.linear(xn, L.qkv, out=qkv)
                ops.rope_kv_write(qkv, positions, row_req, self.kv.block_table, m.inv_freq, cache, c.q_heads, c.kv_heads,
                                  c.head_dim)
                if self.tc_attn and chunk_slot is not None and pos0 is not None:
                    ops.attn_prefill_tc(qkv, qkv.stride(0), cache, self.kv.block_table[chunk_slot], pos0, c.q_heads,
                                        c.kv_heads, c.head_dim, self.scale, out=attn, rows=rows)
                elif self.tc_attn and rows <= 16:
                    ops.attn_decode_tc(qkv, qkv.stride(0), cache, self.kv.block_table, row_req, positions, c.q_heads,
                                       c.kv_heads, c.head_dim, self.scale, splits=self._decode_splits(rows),
                                       scratch=self.att_scratch, out=attn)
                else:
                    ops.attn_decode(qkv, qkv.stride(0), cache, self.kv.block_table, row_req, positions, c.q_heads,
                                    c.kv_heads, c.head_dim, self.scale, out=attn)
                ops.linear(attn, L.o, out=delta)
            have = True
            ops.rmsnorm(x, L.post_norm, c.eps, delta=delta, out=xn)
            self._ffn(i, L, xn, delta)
        ops.rmsnorm(x, m.final_norm, c.eps, delta=delta, out=xn)
        sel = xn if all_logits else xn[rows - 1:rows]
        return ops.gemm_tc(sel, m.head, out32=self.logits[:sel.shape[0]])

    @torch.no_grad()
    def prefill(self, slot: int, tokens: List[int], chunk: int = 256) -> torch.Tensor:
        """Appends `tokens` to request `slot`; returns the logits of the last token [1, V]."""
        start = self.lengths[slot]
        assert self.kv.reserve(slot, start + len(tokens)), "KV pool exhausted"
        out = None
        for o in range(0, len(tokens), chunk):
            part = tokens[o:o + chunk]
            t = torch.tensor(part, dtype=torch.int32, device=self.dev)
            pos = torch.arange(start + o, start + o + len(part), dtype=torch.int32, device=self.dev)
            req = torch.full((len(part),), slot, dtype=torch.int32, device=self.dev)
            out = self.forward(t, pos, req, chunk_slot=slot, all_logits=False, pos0=start + o)
        self.lengths[slot] = start + len(tokens)
        return out

    def _decode_rows(self, slots: List[int], tokens: List[int], positions: List[int]) -> torch.Tensor:
        """One decode pass.  On a GPU the pass is captured once per batch width into a CUDA graph over static id /
        position / request tensors and replayed (a pass is hundreds of small launches; replay removes the host's
        launch cost from every step); `use_graphs = False` launches kernel by kernel."""
        b = len(slots)
        host = torch.tensor([tokens, positions, slots], dtype=torch.int32)
        if not (self.use_graphs and torch.device(self.dev).type == "cuda"):
            d = host.to(self.dev)
            return self.forward(d[0], d[1], d[2])
        st = self._static.get(b)
        if st is None:
            st = self._static[b] = torch.zeros(3, b, dtype=torch.int32, device=self.dev)
        st.copy_(host, non_blocking=True)
        g = self._graphs.get(b)
        if g is None:
            # warm-up outside capture (lazy kernel attributes, workspaces); state-carrying layers are advanced by it,
            # so their state is saved before and put back after: only replays move the model forward
            saved = [t.clone() for t in self._state_tensors()]
            side = torch.cuda.Stream()
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                self.forward(st[0], st[1], st[2])
            torch.cuda.current_stream().wait_stream(side)
            torch.cuda.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                out = self.forward(st[0], st[1], st[2])
            for t, s0 in zip(self._state_tensors(), saved):
                t.copy_(s0)
            g = self._graphs[b] = (graph, out)
        graph, out = g
        graph.replay()
        return out

    @torch.no_grad()
    def decode(self, slots: List[int], tokens: List[int]) -> torch.Tensor:
        """One token for every listed request; returns logits [len(slots), V]."""
        for s in slots:
            assert self.kv.reserve(s, self.lengths[s] + 1), "KV pool exhausted"
        out = self._decode_rows(slots, tokens, [self.lengths[s] for s in slots])
        for s in slots:
            self.lengths[s] += 1
        return out
