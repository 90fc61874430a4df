"""Hybrid decoder family: Gated DeltaNet layers with a full-attention GQA layer every `full_every` layers, dense or
mixture-of-experts feed-forward blocks, and an optional multi-token-prediction (MTP) head for speculative decoding.

``HybridModel.forward_reference`` is the PyTorch oracle (whole sequences, no cache); ``HybridRunner`` executes the
same model with the sm_100a kernels: paged FP8 KV for the attention layers, per-slot recurrent state for the GDN
layers, grouped NVFP4 expert GEMMs for the MoE blocks.  Prefill chunks of one request and batches of single decode
tokens share one code path.
MTP: depth-1 head  h' = block( W_p [norm(h_t) ; norm(embed(x_{t+1}))] ),  logits = lm_head(norm(h')) predicts
x_{t+2}; its proposals are verified by the target model in one pass (`rt.spec_judge`).
(reference counterparts: src/models/qwen/model35.cpp run_rows:2066-2399, glm/mtp.cpp; lines 1934-2123 of the reference tree's top-level design document.)
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
    def random_init(cfg: HybridConfig, device, seed: int = 0, std: float = 0.05, fmt: str = "bf16", ep_rank: int = 0,
                    ep_size: int = 1) -> "HybridModel":
        """ep_size > 1 (expert parallelism): this rank keeps its contiguous block of every MoE layer's experts (and a copy
        of the shared expert); the mixers, norms, embeddings and the head are replicated."""
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
                                               fmt="nvfp4" if torch.device(device).type == "cuda" else "bf16",
                                               ep_rank=ep_rank, ep_size=ep_size, shared_everywhere=ep_size > 1)
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
        # recurrent state of all GDN layers in two pools (layer-major), so one kernel commits a speculative step
        gc = c.gdn_cfg()
        gdn_ids = [i for i in range(c.layers) if not c.is_full(i)]
        self.gdn_index = {i: j for j, i in enumerate(gdn_ids)}
        self.ssm_pool = torch.zeros(max(len(gdn_ids), 1), slots, gc.v_heads, gc.dk, gc.dv, dtype=torch.float32, device=device)
        self.conv_pool = torch.zeros(max(len(gdn_ids), 1), slots, gc.conv_width - 1, gc.conv_channels, dtype=torch.float32,
                                     device=device)
        self.gdn_state = {i: GdnState(gc, slots, device, conv=self.conv_pool[j], ssm=self.ssm_pool[j])
                          for i, j in self.gdn_index.items()}
        self.gdn = {i: GdnLayer(model.layers[i].gdn, max_rows, device) for i in self.gdn_state}
        self.full_index = {i: j for j, i in enumerate(i for i in range(c.layers) if c.is_full(i))}
        self.moe_wide, self._moe_pool = {}, {}
        # expert parallelism (see MlaMoeRunner): MoE layers holding a block of the experts go through the all-to-all
        self.ep, self.ep_small = {}, {}
        first = next((L.moe for L in model.layers if L.moe is not None), None)
        if first is not None and (first.e_end or first.cfg.experts) - first.e_begin < first.cfg.experts:
            from ..parallel.ep import EpMoE
            comm, pool, pool_small = None, {}, {}
            for i, L in enumerate(model.layers):
                if L.moe is not None:
                    self.ep[i] = EpMoE(L.moe, max_rows, device, comm=comm, pool=pool)
                    comm = comm or (self.ep[i].comm, self.ep[i].world, self.ep[i].rank, self.ep[i]._blob)
                    self.ep_small[i] = EpMoE(L.moe, 16, device, comm=comm, pool=pool_small) if max_rows > 16 else self.ep[i]
        self.moe = {i: MoEBlock(L.moe, min(max_rows, 16), device) for i, L in enumerate(model.layers)
                    if L.moe is not None and L.moe.gu_q is not None and not self.ep}
        self.slots = slots
        self.spec_rows = 0          # rows per speculative run (1 + draft depth); 0 = speculation off
        if slots > 16:
            self._ensure_wide()
        e = lambda *s: torch.empty(*s, dtype=BF, device=device)
        H, d = c.hidden, c.head_dim
        self.x, self.xn, self.delta = e(max_rows, H), e(max_rows, H), e(max_rows, H)
        self.qkv = e(max_rows, (c.q_heads + 2 * c.kv_heads) * d)
        self.attn = e(max_rows, c.q_heads * d)
        self.logits = torch.empty(max_rows, c.vocab, dtype=torch.float32, device=device)
        self.lengths = [0] * slots
        self.scale = 1.0 / math.sqrt(d)
        # decode-width passes: NVFP4 linears on the block-scaled path (three-term activations from the norm kernels); off
        # under speculation, whose verify rows must see the arithmetic of plain rows at every batch width
        self.decode_fp4, self.dq = True, ops.DecodeQuant(device)
        self.use_graphs, self._graphs, self._static = True, {}, {}
        self.pdl_graphs = True      # programmatic-dependent-launch edges between this library's kernels in captured passes
        # tensor-core attention (FP8 cache as stored): head_dim 128 / 256, up to 8 query heads per kv head
        self.tc_attn = (torch.device(device).type == "cuda" and d in (128, 256)
                        and c.q_heads // c.kv_heads in (1, 2, 4, 8))
        self.max_splits = 32
        if self.tc_attn:
            r = min(max_rows, 32)
            self.att_scratch = (torch.empty(r * c.q_heads * self.max_splits * 2, dtype=torch.float32, device=device),
                                torch.empty(r * c.q_heads * self.max_splits * d, dtype=torch.float32, device=device))

    def _ensure_wide(self) -> None:
        """Decode blocks for 17..32 rows (more than 16 live requests, or speculative verify rows): the same kernels as
        the 16-row blocks with a 32-row token tile, so a row's arithmetic does not depend on how many rows share its
        pass.  Their large buffers are shared by all layers."""
        if self.moe_wide or self.max_rows <= 16:
            return
        wide = min(self.max_rows, 32)
        self.moe_wide = {i: MoEBlock(self.m.layers[i].moe, wide, self.dev, pool=self._moe_pool) for i in self.moe}

    def _decode_splits(self, rows: int) -> int:
        """KV splits of a decode pass: enough CTAs (kv heads x rows x splits) to cover the SMs; fixed per batch width,
        so a captured pass stays valid at every context length (a split past the end writes an empty partial)."""
        if rows > 32:
            return 1
        if self.spec_rows:
            rows = 1      # verify rows must fold their KV range exactly like a plain decode row does
        return max(1, min(self.max_splits, -(-160 // (self.c.kv_heads * rows))))

    def _state_tensors(self):
        """Tensors a decode pass updates in place besides the KV cache (recurrent layers' state)."""
        return [self.conv_pool, self.ssm_pool]

    def reset(self, slot: int) -> None:
        self.kv.release(slot)
        self.lengths[slot] = 0
        if self.spec_rows:
            self.mtp_kv.release(slot)
            self.mtp_prev[slot], self.mtp_tok[slot], self.mtp_len[slot] = None, [], 0
        for st in self.gdn_state.values():
            st.reset(slot)

    def _ffn(self, i: int, L: HybridLayer, xn: torch.Tensor, out: torch.Tensor, xa=None) -> None:
        if L.moe is not None and i in self.ep:
            (self.ep_small[i] if xn.shape[0] <= 16 else self.ep[i]).forward(xn, out=out)
            return
        if L.moe is not None:
            blk = self.moe.get(i)
            wide = self.moe_wide.get(i)
            if blk is not None and xn.shape[0] <= blk.max_rows:
                blk.forward(xn, out, xa=xa if (xa is not None and blk.bn == xa.bn and blk.terms == xa.terms) else None)
            elif wide is not None and xn.shape[0] <= wide.max_rows:
                wide.forward(xn, out)
            elif blk is not None:
                out.copy_(blk.forward_gathered(xn))
            else:
                out.copy_(moe_reference(xn, L.moe))
            return
        if xa is not None and self.dq.usable(xn.shape[0], L.gate_up, L.down):
            ops.gemm_fp4(self.dq.swiglu(ops.gemm_fp4(xa, L.gate_up), tag="f"), L.down, out=out)
            return
        ops.linear(ops.swiglu(ops.linear(xn, L.gate_up)), L.down, out=out)

    @torch.no_grad()
    def forward(self, tokens: torch.Tensor, positions: torch.Tensor, row_req: torch.Tensor, chunk_slot: Optional[int] = None,
                all_logits: bool = True, pos0: Optional[int] = None, seg: int = 0, snap: bool = False) -> torch.Tensor:
        """tokens / positions / row_req: int32 [rows] on the device.  chunk_slot given: the rows are consecutive
        tokens of that request starting at position pos0 (prefill chunk); otherwise one decode token per row.
        seg > 0: the rows are runs of `seg` consecutive tokens per request (speculative verify); snap: the recurrent
        layers save their state after every row.  Returns fp32 logits [rows, V]; the residual stream before the final
        norm (the MTP head's input) stays in self.x[:rows]."""
        m, c = self.m, self.c
        rows = tokens.shape[0]
        x, xn, delta = self.x[:rows], self.xn[:rows], self.delta[:rows]
        ops.embed_gather(tokens, m.embed, out=x)
        have = False
        dq = self.dq
        for i, L in enumerate(m.layers):
            w_in = L.gdn.in_proj if L.gdn is not None else L.qkv
            fast = self.decode_fp4 and not self.spec_rows and chunk_slot is None and dq.usable(rows, w_in)
            xa = None
            if fast:
                xa = dq.norm(x, L.in_norm, c.eps, delta=delta if have else None, x_out=xn, tag="h")
            else:
                ops.rmsnorm(x, L.in_norm, c.eps, delta=delta if have else None, out=xn)
            if L.gdn is not None:
                j = self.gdn_index[i]
                self.gdn[i].forward(xn, self.gdn_state[i], delta, slot=chunk_slot or 0,
                                    row_slot=None if chunk_slot is not None else row_req, seg=seg,
                                    snap=(self.conv_snap[j], self.ssm_snap[j]) if snap else None, xa=xa, dq=dq)
            else:
                cache = self.kv.layers[self.full_index[i]]
                qkv, attn = self.qkv[:rows], self.attn[:rows]
                if fast:
                    ops.gemm_fp4(xa, L.qkv, out=qkv)
                else:
                    ops.linear(xn, L.qkv, out=qkv)
                ops.rope_kv_write(qkv, positions, row_req, self.kv.block_table, m.inv_freq, cache, c.q_heads, c.kv_heads,
                                  c.head_dim)
                if self.tc_attn and chunk_slot is not None and pos0 is not None:
                    ops.attn_prefill_tc(qkv, qkv.stride(0), cache, self.kv.block_table[chunk_slot], pos0, c.q_heads,
                                        c.kv_heads, c.head_dim, self.scale, out=attn, rows=rows)
                elif self.tc_attn and rows <= 32:
                    ops.attn_decode_tc(qkv, qkv.stride(0), cache, self.kv.block_table, row_req, positions, c.q_heads,
                                       c.kv_heads, c.head_dim, self.scale, splits=self._decode_splits(rows),
                                       scratch=self.att_scratch, out=attn)
                else:
                    ops.attn_decode(qkv, qkv.stride(0), cache, self.kv.block_table, row_req, positions, c.q_heads,
                                    c.kv_heads, c.head_dim, self.scale, out=attn)
                if fast and dq.usable(rows, L.o):
                    ops.gemm_fp4(dq.plain(attn, "a"), L.o, out=delta)
                else:
                    ops.linear(attn, L.o, out=delta)
            have = True
            xa = None
            if fast:
                xa = dq.norm(x, L.post_norm, c.eps, delta=delta, x_out=xn, tag="h")
            else:
                ops.rmsnorm(x, L.post_norm, c.eps, delta=delta, out=xn)
            self._ffn(i, L, xn, delta, xa=xa)
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
            if self.spec_rows:
                self._mtp_after_prefill(slot, self.x[:len(part)].clone(), part, start + o)
        self.lengths[slot] = start + len(tokens)
        if self.spec_rows:
            self.mtp_tok[slot] = []
        return out

    def _decode_rows(self, slots: List[int], tokens: List[int], positions: List[int], seg: int = 0) -> torch.Tensor:
        """One decode pass.  On a GPU the pass is captured once per batch width into a CUDA graph over static id /
        position / request tensors and replayed (a pass is hundreds of small launches; replay removes the host's
        launch cost from every step); `use_graphs = False` launches kernel by kernel."""
        b = len(slots)
        snap = seg > 0
        on_dev = isinstance(tokens, torch.Tensor)          # speculative drafts never visit the host
        if on_dev:
            host = torch.tensor([positions, slots], dtype=torch.int32)
        else:
            host = torch.tensor([tokens, positions, slots], dtype=torch.int32)
        if not (self.use_graphs and torch.device(self.dev).type == "cuda"):
            d = host.to(self.dev)
            if on_dev:
                return self.forward(tokens, d[0], d[1], seg=seg, snap=snap)
            return self.forward(d[0], d[1], d[2], seg=seg, snap=snap)
        key = (b, seg)
        st = self._static.get(key)
        if st is None:
            st = self._static[key] = torch.zeros(3, b, dtype=torch.int32, device=self.dev)
        if on_dev:
            st[0].copy_(tokens)
            st[1:].copy_(host, non_blocking=True)
        else:
            st.copy_(host, non_blocking=True)
        g = self._graphs.get(key)
        if g is None:
            # warm-up outside capture (lazy kernel attributes, workspaces); state-carrying layers are advanced by it,
            # so their state is saved before and put back after: only replays move the model forward
            saved = [t.clone() for t in self._state_tensors()]
            side = torch.cuda.Stream()
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                self.forward(st[0], st[1], st[2], seg=seg, snap=snap)
            torch.cuda.current_stream().wait_stream(side)
            torch.cuda.synchronize()
            from ..engine.graph import capture_with_pdl
            graph, out, _ = capture_with_pdl(lambda: self.forward(st[0], st[1], st[2], seg=seg, snap=snap), self.pdl_graphs)
            for t, s0 in zip(self._state_tensors(), saved):
                t.copy_(s0)
            g = self._graphs[key] = (graph, out)
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

    # ------------------------------------------------------------------ multi-token prediction: draft, verify, commit
    def enable_spec(self, depth: int) -> None:
        """Turn on speculative decoding with `depth` drafts per step from the MTP head (1 <= depth <= 3).  Call before the
        first prefill: the head keeps its own one-layer KV cache, filled alongside the model's.
        (reference counterparts: src/models/qwen/model35.cpp:1909 mtp_run_rows, src/engine/speculative.hpp:155.)"""
        from ..engine.kv_cache import PagedKV

        m, c = self.m, self.c
        assert m.mtp_layer is not None, "the model has no MTP head"
        assert 1 <= depth <= 3 and all(n == 0 for n in self.lengths)
        V = depth + 1
        self.spec_rows = V
        rows = self.slots * V
        gc = c.gdn_cfg()
        Lg = self.ssm_pool.shape[0]
        self.ssm_snap = torch.zeros(Lg, rows, gc.v_heads, gc.dk, gc.dv, dtype=torch.float32, device=self.dev)
        self.conv_snap = torch.zeros(Lg, rows, gc.conv_width - 1, gc.conv_channels, dtype=torch.float32, device=self.dev)
        self.mtp_kv = PagedKV(1, c.kv_heads, c.head_dim, self.kv.num_blocks, self.slots, self.kv.max_blocks, c.page, True,
                              self.dev)
        L = m.mtp_layer
        self.mtp_moe = MoEBlock(L.moe, 16, self.dev) if (L.moe is not None and L.moe.gu_q is not None) else None
        self.mtp_moe_wide = None
        if rows > 16:
            self._ensure_wide()
            if self.mtp_moe is not None and self.max_rows > 16:
                self.mtp_moe_wide = MoEBlock(L.moe, min(self.max_rows, 32), self.dev, pool=self._moe_pool)
        self.mtp_prev = [None] * self.slots      # main-model hidden rows whose MTP pair still waits for its next token
        self.mtp_tok = [[] for _ in range(self.slots)]   # tokens after those rows, the newest excepted (it is the pending one)
        self.mtp_len = [0] * self.slots          # MTP cache filled for positions < mtp_len
        i32 = dict(dtype=torch.int32, device=self.dev)
        self.n_acc, self.emitted = torch.zeros(self.slots, **i32), torch.zeros(self.slots * V, **i32)
        self._graphs.clear()                     # decode splits are pinned once speculation is on
        ops.PIN_SPLIT_ROWS = True                # (process-wide: plain passes of this process pick the same splits)

    def _mtp_rows(self, hidden: torch.Tensor, next_tokens: torch.Tensor, positions: torch.Tensor, row_req: torch.Tensor,
                  chunk_slot: Optional[int] = None, pos0: Optional[int] = None):
        """MTP head over the pairs (hidden_t, token_{t+1}) at MTP positions `positions` (its own KV cache is appended at
        those positions).  Returns (fp32 logits [rows, V] for token_{t+2}, the head's residual stream [rows, H])."""
        m, c = self.m, self.c
        rows = hidden.shape[0]
        L = m.mtp_layer
        hn = ops.rmsnorm(hidden, m.mtp_norm_h, c.eps)
        emb = ops.embed_gather(next_tokens, m.embed, out=torch.empty(rows, c.hidden, dtype=BF, device=self.dev))
        en = ops.rmsnorm(emb, m.mtp_norm_e, c.eps)
        x = ops.linear(torch.cat([hn, en], -1), m.mtp_proj)
        xn = ops.rmsnorm(x, L.in_norm, c.eps)
        cache = self.mtp_kv.layers[0]
        qkv = ops.linear(xn, L.qkv)
        ops.rope_kv_write(qkv, positions, row_req, self.mtp_kv.block_table, m.inv_freq, cache, c.q_heads, c.kv_heads, c.head_dim)
        if self.tc_attn and chunk_slot is not None and pos0 is not None and rows > 32:
            attn = ops.attn_prefill_tc(qkv, qkv.stride(0), cache, self.mtp_kv.block_table[chunk_slot], pos0, c.q_heads,
                                       c.kv_heads, c.head_dim, self.scale, rows=rows)
        elif self.tc_attn and rows <= 32:
            attn = ops.attn_decode_tc(qkv, qkv.stride(0), cache, self.mtp_kv.block_table, row_req, positions, c.q_heads,
                                      c.kv_heads, c.head_dim, self.scale, splits=self._decode_splits(rows),
                                      scratch=self.att_scratch)
        else:
            attn = ops.attn_decode(qkv, qkv.stride(0), cache, self.mtp_kv.block_table, row_req, positions, c.q_heads,
                                   c.kv_heads, c.head_dim, self.scale)
        delta = ops.linear(attn, L.o)
        xn = ops.rmsnorm(x, L.post_norm, c.eps, delta=delta)
        if L.moe is not None:
            if self.mtp_moe is not None and rows <= self.mtp_moe.max_rows:
                self.mtp_moe.forward(xn, delta)
            elif self.mtp_moe_wide is not None and rows <= self.mtp_moe_wide.max_rows:
                self.mtp_moe_wide.forward(xn, delta)
            elif self.mtp_moe is not None:
                delta = self.mtp_moe.forward_gathered(xn)
            else:
                delta = moe_reference(xn, L.moe)
        else:
            delta = ops.linear(ops.swiglu(ops.linear(xn, L.gate_up)), L.down)
        xn = ops.rmsnorm(x, m.final_norm, c.eps, delta=delta)
        logits = ops.gemm_tc(xn, m.head, out32=torch.empty(rows, c.vocab, dtype=torch.float32, device=self.dev))
        return logits, x

    def _mtp_after_prefill(self, slot: int, hidden: torch.Tensor, tokens: List[int], start: int) -> None:
        """Feed the MTP cache with the pairs a prefill chunk completes: (hidden_{t}, token_{t+1}) for every t whose next
        token is known; the chunk's last hidden row waits for the next token."""
        T = hidden.shape[0]
        rows, toks, p0 = hidden[:T - 1], tokens[1:], start
        if self.mtp_prev[slot] is not None:
            rows, toks, p0 = torch.cat([self.mtp_prev[slot], rows]), tokens, start - self.mtp_prev[slot].shape[0]
        n = rows.shape[0]
        if n:
            assert self.mtp_kv.reserve(slot, p0 + n), "MTP KV pool exhausted"
            t = torch.tensor(toks, dtype=torch.int32, device=self.dev)
            pos = torch.arange(p0, p0 + n, dtype=torch.int32, device=self.dev)
            req = torch.full((n,), slot, dtype=torch.int32, device=self.dev)
            self._mtp_rows(rows.contiguous(), t, pos, req, chunk_slot=slot, pos0=p0)
            self.mtp_len[slot] = p0 + n
        self.mtp_prev[slot] = hidden[T - 1:T].clone()

    @torch.no_grad()
    def spec_step(self, slots: List[int], pending: List[int], drafts: Optional[List[List[int]]] = None) -> List[List[int]]:
        """One speculative step for the listed requests.  pending[i]: the token emitted last for slots[i] (not yet in the
        caches).  Drafts come from the MTP head (or from `drafts`, depth tokens per request, for tests).  Returns the new
        tokens of every request (1 .. depth + 1 of them); the last one is its new pending token.  Greedy: the emitted
        sequence is the one plain decoding emits."""
        V, R = self.spec_rows, len(slots)
        assert V >= 2, "enable_spec first"
        depth = V - 1
        dev = self.dev
        i32 = dict(dtype=torch.int32, device=dev)
        if drafts is None:
            # draft pass 0: every pair that waits (hidden rows of the last step, their next tokens ending in the pending one)
            hid, toks, pos, req, last = [], [], [], [], []
            for s, p in zip(slots, pending):
                h = self.mtp_prev[s]
                n = h.shape[0]
                known = self.mtp_tok[s][:n - 1]
                hid.append(h)
                toks += list(known) + [p]
                p0 = self.lengths[s] - n
                pos += list(range(p0, p0 + n))
                req += [s] * n
                last.append(len(toks) - 1)
                assert self.mtp_kv.reserve(s, self.lengths[s] + V), "MTP KV pool exhausted"
            logits, hm = self._mtp_rows(torch.cat(hid), torch.tensor(toks, **i32), torch.tensor(pos, **i32),
                                        torch.tensor(req, **i32))
            sel = torch.tensor(last, dtype=torch.long, device=dev)
            d = torch.argmax(logits[sel], -1).to(torch.int32)
            cols = [d]
            hm = hm[sel].contiguous()
            rreq = torch.tensor(slots, **i32)
            base = torch.tensor([self.lengths[s] for s in slots], **i32)
            for j in range(1, depth):
                logits, hm = self._mtp_rows(hm, cols[-1], base - 1 + j, rreq)
                cols.append(torch.argmax(logits, -1).to(torch.int32))
            dr = torch.stack(cols, 1)                                   # [R, depth] on the device
        else:
            dr = torch.tensor(drafts, **i32).view(R, depth)
        tok = torch.cat([torch.tensor(pending, **i32).view(R, 1), dr], 1).reshape(-1)        # [R * V]
        for s in slots:
            assert self.kv.reserve(s, self.lengths[s] + V), "KV pool exhausted"
        positions = [self.lengths[s] + i for s in slots for i in range(V)]
        row_slots = [s for s in slots for _ in range(V)]
        req_d = torch.tensor(row_slots, **i32)
        logits = self._decode_rows(row_slots, tok, positions, seg=V)      # tokens stay on the device
        picks = torch.argmax(logits[:R * V], -1).to(torch.int32)
        hidden = self.x[:R * V].clone()
        ops.spec_accept(tok, picks, self.n_acc, self.emitted, R, V)
        ops.spec_commit(self.ssm_pool, self.ssm_snap, self.conv_pool, self.conv_snap, req_d, self.n_acc, R, V)
        host = torch.cat([self.n_acc[:R], self.emitted[:R * V], tok]).tolist()       # the step's one device -> host read
        n_acc, emitted, tok_h = host[:R], host[R:R + R * V], host[R + R * V:]
        out = []
        for r, s in enumerate(slots):
            n = n_acc[r]
            new = emitted[r * V:r * V + n]
            self.lengths[s] += n
            self.mtp_prev[s] = hidden[r * V:r * V + n]
            self.mtp_tok[s] = tok_h[r * V + 1:r * V + n] + [new[-1]]
            out.append(new)
        self.spec_steps = getattr(self, "spec_steps", 0) + R
        self.spec_tokens = getattr(self, "spec_tokens", 0) + sum(len(o) for o in out)
        return out
