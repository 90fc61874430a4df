"""Gated-residual hybrid family (Flash-Next style): `hc` residual branches per token, Gated DeltaNet layers with one
full-attention layer in every `full_every`, dense or mixture-of-experts FFN, hashed bigram embeddings.

Every sub-block (token mixer, FFN) reads one row mixed from the branches through a low-rank sigmoid gate and injects
its output into every branch with a per-branch strength:

    rn      = rmsnorm(R)                                   R: [hc * H] residual branches of the token
    gate    = sigmoid(W_up silu(W_down rn / hc))           [hc * H]
    x       = (1 / hc) sum_i gate_i * rn_i                 [H]      -> y = block(x)
    R_i    += y * 2 sigmoid(<w_inject_i, rn> / hc)

The token embedding is the vocabulary row plus a row of a hashed table indexed by (previous token, token), so a
request remembers its last token between passes.  The full-attention layers are causal GQA over the paged FP8 cache,
dense or (with `qsa`) block-sparse with pooled index keys: every token projects `index_heads` index queries (RMSNorm
with 1 + w, rotary) and one raw index key; when a block of `page` tokens completes, its raw keys are averaged,
normalised and rotated at the block's first position into one compressed key; a row scores every complete visible
block by sum_h relu(<q_h, c_b>) / sqrt(index_dim), keeps the `select_k` best (ties to the lower block) plus its own
incomplete block, and attends only to the tokens of those blocks (one list per row, shared by the kv heads).
Oracle: ``FlashNextModel.forward_reference``; kernels: `gr_gate_act`, `gr_mix_finish`, `gr_combine`, the GDN layer
kernels, rotary + KV append, tcgen05 attention (dense) or `msa_index_prep` (raw keys) / `qsa_compress` / `qsa_select` and
the block-selection form of the paged decode attention (sparse), the MoE block, tensor-core linears.
(reference counterparts: src/models/qwen/forward.cpp, layers.cpp (GR residual, PLE), src/kernels/qwen_gr.cu,
 src/kernels/qsa.hpp (indexer, score, select, listed attention), src/kernels/gdn_chunk.cu, src/models/qwen/moe_layer.cpp.)
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import List, Optional

import torch

from ..ops import core as ops
from ..ops import reference as ref
from ..quant.formats import QuantLinear, quantize
from .gdn import GdnConfig, GdnLayer, GdnState, GdnWeights, gdn_reference
from .moe import MoEBlock, MoEConfig, MoEWeights, moe_reference
from .rows import RowRunner

BF = torch.bfloat16


@dataclass
class QsaConfig:
    index_heads: int = 4
    index_dim: int = 128
    select_k: int = 2            # complete blocks kept per row (the row's own incomplete block comes on top)


@dataclass
class FlashNextConfig:
    layers: int = 4
    hidden: int = 512
    full_every: int = 4
    hc: int = 4                  # residual branches
    gr_rank: int = 128           # width of the low-rank gate
    q_heads: int = 4
    kv_heads: int = 2
    head_dim: int = 128
    gdn_k_heads: int = 2
    gdn_v_heads: int = 4
    gdn_dk: int = 128
    gdn_dv: int = 128
    ffn: int = 1024
    moe: Optional[MoEConfig] = None
    vocab: int = 2048
    ple_rows: int = 4096         # hashed bigram table (0 = none)
    rope_theta: float = 1e4
    eps: float = 1e-6
    page: int = 64               # KV page = the pooled block of the sparse index
    qsa: Optional[QsaConfig] = None

    def is_full(self, i: int) -> bool:
        return (i + 1) % self.full_every == 0

    def gdn_cfg(self) -> GdnConfig:
        return GdnConfig(self.hidden, self.gdn_k_heads, self.gdn_v_heads, self.gdn_dk, self.gdn_dv, 4, self.eps)

    def ple_id(self, prev: int, tok: int) -> int:
        return (prev * 1000003 + tok * 7919 + 12345) % self.ple_rows


@dataclass
class GrSite:
    norm: torch.Tensor           # [hc * H] bf16
    w_down: QuantLinear          # [rank, hc * H]
    w_up: QuantLinear            # [hc * H, rank]
    w_inject: torch.Tensor       # [hc, hc * H] bf16


@dataclass
class FlashNextLayer:
    mix: GrSite
    ffn_site: GrSite
    gdn: Optional[GdnWeights] = None
    qkv: Optional[QuantLinear] = None
    o: Optional[QuantLinear] = None
    gate_up: Optional[QuantLinear] = None
    down: Optional[QuantLinear] = None
    moe: Optional[MoEWeights] = None
    index: Optional[QuantLinear] = None          # [(index_heads + 1) * index_dim, H]: index queries, then the raw key
    index_q_norm: Optional[torch.Tensor] = None  # [index_dim] bf16, applied as 1 + w
    index_k_norm: Optional[torch.Tensor] = None


def qsa_keep_reference(iq: torch.Tensor, raw_k: torch.Tensor, k_norm, inv_freq, page: int, select_k: int, eps: float) -> torch.Tensor:
    """iq [T, ih, di] (normed, rotated), raw_k [T, di] fp32 of one request from position 0 -> bool [T, nblocks]: the
    blocks every row attends to (complete blocks by score, own incomplete block always)."""
    T, ih, di = iq.shape
    nb = (T + page - 1) // page
    full = T // page
    keep = torch.zeros(T, nb, dtype=torch.bool, device=iq.device)
    t = torch.arange(T, device=iq.device)
    if full:
        mean = ref._r(raw_k[:full * page].view(full, page, di).mean(1))
        first = torch.arange(full, device=iq.device) * page
        comp = ref.apply_rope(ref.head_norm(mean.unsqueeze(1), k_norm, eps, True), first, inv_freq, di)[:, 0]     # [full, di]
        s = torch.relu(torch.einsum("thd,bd->thb", iq, comp)).sum(1) / (di ** 0.5)                               # [T, full]
        visible = ((t + 1) // page).view(T, 1)
        s = s.masked_fill(torch.arange(full, device=iq.device).view(1, full) >= visible, float("-inf"))
        order = torch.argsort(-s, dim=-1, stable=True)[:, :select_k]
        picked = torch.zeros(T, full, dtype=torch.bool, device=iq.device)
        picked.scatter_(1, order, True)
        keep[:, :full] = picked & (s > float("-inf"))
    tail = (t + 1) % page != 0
    keep[t[tail], (t // page)[tail]] = True
    return keep


class FlashNextModel:
    def __init__(self, cfg: FlashNextConfig, embed, ple, layers: List[FlashNextLayer], final: GrSite, final_norm,
                 head: QuantLinear, inv_freq):
        self.cfg, self.embed, self.ple, self.layers, self.final, self.final_norm, self.head, self.inv_freq = \
            cfg, embed, ple, layers, final, final_norm, head, inv_freq
        self.inv_idx = None if cfg.qsa is None else ref.rope_inv_freq(cfg.qsa.index_dim, cfg.rope_theta, embed.device)[0]

    @staticmethod
    def random_init(cfg: FlashNextConfig, device, seed: int = 0, std: float = 0.05, fmt: str = "bf16") -> "FlashNextModel":
        g = torch.Generator(device=device)
        g.manual_seed(seed)
        c, H, d = cfg, cfg.hidden, cfg.head_dim
        rnd = lambda *s: torch.randn(*s, device=device, dtype=torch.float32, generator=g)
        lin = lambda n, k: quantize(rnd(n, k) * std, fmt if (k % 256 == 0 or fmt == "bf16") else "bf16")

        def site():
            return GrSite((1 + 0.1 * rnd(c.hc * H)).to(BF), quantize(rnd(c.gr_rank, c.hc * H) * std, "bf16"),
                          quantize(rnd(c.hc * H, c.gr_rank) * std * 4, "bf16"), (rnd(c.hc, c.hc * H) * std).to(BF))

        layers = []
        for i in range(c.layers):
            L = FlashNextLayer(site(), site())
            if c.is_full(i):
                L.qkv, L.o = lin((c.q_heads + 2 * c.kv_heads) * d, H), lin(H, c.q_heads * d)
                if c.qsa is not None:
                    q = c.qsa
                    L.index = quantize(rnd((q.index_heads + 1) * q.index_dim, H) * std * 2, "bf16")
                    L.index_q_norm, L.index_k_norm = (0.1 * rnd(q.index_dim)).to(BF), (0.1 * rnd(q.index_dim)).to(BF)
            else:
                L.gdn = GdnWeights.random_init(c.gdn_cfg(), device, seed=seed * 77 + i, std=std, fmt=fmt)
            if c.moe is not None:
                L.moe = MoEWeights.random_init(c.moe, device, seed=seed * 1000 + i, std=std)
            else:
                L.gate_up, L.down = lin(2 * c.ffn, H), lin(H, c.ffn)
            layers.append(L)
        inv, _ = ref.rope_inv_freq(d, c.rope_theta, device)
        ple = (rnd(c.ple_rows, H) * std).to(BF) if c.ple_rows else None
        return FlashNextModel(cfg, (rnd(c.vocab, H) * std * 4).to(BF), ple, layers, site(), torch.ones(H, device=device, dtype=BF),
                              quantize(rnd(c.vocab, H) * std, "bf16"), inv)

    def ple_ids(self, tokens: List[int], prev: int = 0) -> List[int]:
        out = []
        for t in tokens:
            out.append(self.cfg.ple_id(prev, t))
            prev = t
        return out

    # ------------------------------------------------------------------ oracle
    def _mix_reference(self, s: GrSite, R: torch.Tensor):
        c = self.cfg
        rn = ref.rmsnorm(R, s.norm, c.eps)[0]
        t = ref.gr_gate_act(ref.linear(rn, s.w_down), c.hc)
        return ref.gr_mix_finish(ref.linear(t, s.w_up), rn, c.hc), rn

    def forward_reference(self, tokens: torch.Tensor) -> torch.Tensor:
        """fp32 logits [T, V] of one request from position 0."""
        c, d = self.cfg, self.cfg.head_dim
        dev = self.embed.device
        T = tokens.numel()
        pos = torch.arange(T, device=dev)
        x = ref.embed_gather(tokens.to(dev), self.embed)
        if self.ple is not None:
            ids = torch.tensor(self.ple_ids(tokens.tolist()), device=dev)
            x = (x.float() + ref.embed_gather(ids, self.ple).float()).to(BF)
        R = x.repeat(1, c.hc).contiguous()
        nq, nkv = c.q_heads * d, c.kv_heads * d

        def site(s: GrSite, block):
            nonlocal R
            xin, rn = self._mix_reference(s, R)
            R = ref.gr_combine(R, rn, s.w_inject, block(xin), c.hc)

        def attention(L, xin):
            qkv = ref.linear(xin, L.qkv).float()
            q = ref.apply_rope(qkv[:, :nq].view(T, c.q_heads, d), pos, self.inv_freq, d)
            k = ref.apply_rope(qkv[:, nq:nq + nkv].view(T, c.kv_heads, d), pos, self.inv_freq, d)
            v = ref._r(qkv[:, nq + nkv:].view(T, c.kv_heads, d))
            if c.qsa is None:
                a = ref.attention(q, k, v, 1.0 / math.sqrt(d), causal_offset=0)
                return ref.linear(ref.act(a.reshape(T, nq)), L.o)
            qs = c.qsa
            iqk = ref.linear(xin, L.index).float().view(T, qs.index_heads + 1, qs.index_dim)
            iq = ref.apply_rope(ref.head_norm(iqk[:, :qs.index_heads], L.index_q_norm, c.eps, True), pos, self.inv_idx, qs.index_dim)
            keep = qsa_keep_reference(iq, iqk[:, qs.index_heads], L.index_k_norm, self.inv_idx, c.page, qs.select_k, c.eps)
            kq, ks = ref.quant_kv_fp8(k)
            vq, vs = ref.quant_kv_fp8(v)
            k = kq.view(torch.float8_e4m3fn).float() * ks.unsqueeze(-1)
            v = vq.view(torch.float8_e4m3fn).float() * vs.unsqueeze(-1)
            g = c.q_heads // c.kv_heads
            t = torch.arange(T, device=dev)
            allowed = keep[:, t // c.page] & (t.view(1, T) <= t.view(T, 1))                   # [T, T]
            s = torch.einsum("qhd,khd->hqk", q, k.repeat_interleave(g, 1)) / math.sqrt(d)
            s = s.masked_fill(~allowed.unsqueeze(0), float("-inf"))
            a = torch.einsum("hqk,khd->qhd", torch.nan_to_num(torch.softmax(s, -1)), v.repeat_interleave(g, 1))
            return ref.linear(ref.act(a.reshape(T, nq)), L.o)

        for L in self.layers:
            if L.gdn is not None:
                cs = torch.zeros(3, c.gdn_cfg().conv_channels, device=dev)
                ss = torch.zeros(c.gdn_v_heads, c.gdn_dk, c.gdn_dv, device=dev)
                site(L.mix, lambda xin: gdn_reference(xin, L.gdn, cs, ss))
            else:
                site(L.mix, lambda xin: attention(L, xin))
            if L.moe is not None:
                site(L.ffn_site, lambda xin: moe_reference(xin, L.moe))
            else:
                site(L.ffn_site, lambda xin: ref.linear(ref.swiglu(ref.linear(xin, L.gate_up)), L.down))
        xin, _ = self._mix_reference(self.final, R)
        return ref.linear(ref.rmsnorm(xin, self.final_norm, c.eps)[0], self.head, out_fp32=True)


class FlashNextRunner(RowRunner):
    def __init__(self, model: FlashNextModel, max_rows: int, slots: int, max_seq_len: int, device):
        c = model.cfg
        self.m, self.c = model, c
        n_full = sum(1 for i in range(c.layers) if c.is_full(i))
        self._init_rows(slots, device, kv_layers=max(n_full, 1), kv_heads=c.kv_heads, q_heads=c.q_heads, head_dim=c.head_dim,
                        page=c.page, max_seq_len=max_seq_len, max_rows=max_rows)
        gc = c.gdn_cfg()
        self.full_index = {i: j for j, i in enumerate(i for i in range(c.layers) if c.is_full(i))}
        self.gdn_index = {i: j for j, i in enumerate(i for i in range(c.layers) if not c.is_full(i))}
        Lg = max(len(self.gdn_index), 1)
        self.ssm_pool = torch.zeros(Lg, slots, gc.v_heads, gc.dk, gc.dv, dtype=torch.float32, device=device)
        self.conv_pool = torch.zeros(Lg, slots, gc.conv_width - 1, gc.conv_channels, dtype=torch.float32, device=device)
        self.gdn_state = {i: GdnState(gc, slots, device, conv=self.conv_pool[j], ssm=self.ssm_pool[j])
                          for i, j in self.gdn_index.items()}
        self.gdn = {i: GdnLayer(model.layers[i].gdn, max_rows, device) for i in self.gdn_index}
        pool = {}
        self.moe = {i: MoEBlock(L.moe, min(max_rows, 16), device, pool=pool) for i, L in enumerate(model.layers)
                    if L.moe is not None and L.moe.gu_q is not None}
        e = lambda *s: torch.empty(*s, dtype=BF, device=device)
        H = c.hidden
        self.R, self.rn, self.logits_g = e(max_rows, c.hc * H), e(max_rows, c.hc * H), e(max_rows, c.hc * H)
        self.t = e(max_rows, c.gr_rank)
        self.x, self.y = e(max_rows, H), e(max_rows, H)
        self.qkv = e(max_rows, (c.q_heads + 2 * c.kv_heads) * c.head_dim)
        self.attn = e(max_rows, c.q_heads * c.head_dim)
        self.last_token = [0] * slots
        if c.qsa is not None:
            q, blocks = c.qsa, self.kv.layers[0].k.shape[0]
            self.idx_raw = [torch.zeros(blocks, c.page, q.index_dim, dtype=BF, device=device) for _ in self.full_index]
            self.idx_comp = [torch.zeros(blocks, q.index_dim, dtype=BF, device=device) for _ in self.full_index]
            self.iqk = e(max_rows, (q.index_heads + 1) * q.index_dim)
            self.sel = torch.empty(max_rows, c.kv_heads, q.select_k + 1, dtype=torch.int32, device=device)
            self.max_sel = (max_seq_len + c.page - 1) // c.page + 1
            self.sp_splits = 8
            self.sp_scratch = (torch.empty(max_rows * c.q_heads * self.sp_splits * 2, dtype=torch.float32, device=device),
                               torch.empty(max_rows * c.q_heads * self.sp_splits * c.head_dim, dtype=torch.float32, device=device))

    def _state_tensors(self):
        return [self.conv_pool, self.ssm_pool]

    def _reset_state(self, slot: int) -> None:
        self.ssm_pool[:, slot].zero_()
        self.conv_pool[:, slot].zero_()
        self.last_token[slot] = 0

    def _extra_rows(self, slots, tokens, prefill_slot=None):
        if self.m.ple is None:
            return []
        # the previous token of every row; the bigram hash and the table gather run on the device
        if prefill_slot is not None:
            return [[self.last_token[prefill_slot]] + list(tokens[:-1])]
        return [[self.last_token[s] for s in slots]]

    def _note_tokens(self, slot, tokens):
        self.last_token[slot] = tokens[-1]

    def _sparse_attention(self, j: int, L: FlashNextLayer, xin, qkv, positions, row_req, attn) -> None:
        c, q, rows = self.c, self.c.qsa, xin.shape[0]
        cache, bt = self.kv.layers[j], self.kv.block_table
        iqk, sel = self.iqk[:rows], self.sel[:rows]
        ops.rope_kv_write(qkv, positions, row_req, bt, self.m.inv_freq, cache, c.q_heads, c.kv_heads, c.head_dim)
        ops.linear(xin, L.index, out=iqk)
        ops.msa_index_prep(iqk, positions, row_req, bt, self.m.inv_idx, L.index_q_norm, None, self.idx_raw[j], q.index_heads,
                           q.index_dim, q.index_dim, c.eps, one_plus_w=True, raw_key=True)
        ops.qsa_compress(self.idx_raw[j], self.idx_comp[j], positions, row_req, bt, self.m.inv_idx, L.index_k_norm, q.index_dim,
                         c.eps, one_plus_w=True)
        ops.qsa_select(iqk, self.idx_comp[j], bt, row_req, positions, q.index_heads, q.index_dim, c.page, q.select_k,
                       self.max_sel, copies=c.kv_heads, out=sel)
        fn = ops.attn_decode_tc if (self.tc_attn and rows <= 32) else ops.attn_decode
        fn(qkv, qkv.stride(0), cache, bt, row_req, positions, c.q_heads, c.kv_heads, c.head_dim, self.att_scale,
           splits=self.sp_splits, scratch=self.sp_scratch, out=attn, sel=sel, sel_block=c.page)

    def _mix(self, s: GrSite, rows: int) -> torch.Tensor:
        c = self.c
        rn = ops.rmsnorm(self.R[:rows], s.norm, c.eps, out=self.rn[:rows])
        t = ops.gr_gate_act(ops.linear(rn, s.w_down, out=self.t[:rows]), c.hc)
        logits = ops.linear(t, s.w_up, out=self.logits_g[:rows])
        return ops.gr_mix_finish(logits, rn, c.hc)

    def _site(self, s: GrSite, rows: int, block) -> None:
        xin = self._mix(s, rows)
        block(xin, self.y[:rows])
        ops.gr_combine(self.R[:rows], self.rn[:rows], s.w_inject, self.y[:rows], self.c.hc)

    def _ffn(self, i: int, L: FlashNextLayer, xin: torch.Tensor, out: torch.Tensor) -> None:
        if L.moe is None:
            ops.linear(ops.swiglu(ops.linear(xin, L.gate_up)), L.down, out=out)
            return
        blk = self.moe.get(i)
        if blk is not None and xin.shape[0] <= blk.max_rows:
            blk.forward(xin, out)
        elif blk is not None:
            out.copy_(blk.forward_gathered(xin))
        else:
            out.copy_(moe_reference(xin, L.moe))

    @torch.no_grad()
    def forward(self, tokens, positions, row_req, chunk_slot=None, all_logits=True, pos0=None, extra=None):
        m, c = self.m, self.c
        rows = tokens.shape[0]
        x = ops.embed_gather(tokens, m.embed, out=self.x[:rows])
        if m.ple is not None:
            ops.ple_embed_add(tokens, extra[0], m.ple, x)
        self.R[:rows].view(rows, c.hc, c.hidden).copy_(x.unsqueeze(1).expand(rows, c.hc, c.hidden))
        for i, L in enumerate(m.layers):
            if L.gdn is not None:
                self._site(L.mix, rows, lambda xin, out: self.gdn[i].forward(
                    xin, self.gdn_state[i], out, slot=chunk_slot or 0, row_slot=None if chunk_slot is not None else row_req))
            else:
                def attention(xin, out):
                    qkv, attn = self.qkv[:rows], self.attn[:rows]
                    ops.linear(xin, L.qkv, out=qkv)
                    if c.qsa is None:
                        self._attention_rows(self.full_index[i], qkv, positions, row_req, m.inv_freq, chunk_slot, pos0, attn)
                    else:
                        self._sparse_attention(self.full_index[i], L, xin, qkv, positions, row_req, attn)
                    ops.linear(attn, L.o, out=out)
                self._site(L.mix, rows, attention)
            self._site(L.ffn_site, rows, lambda xin, out: self._ffn(i, L, xin, out))
        xn = ops.rmsnorm(self._mix(m.final, rows), m.final_norm, c.eps)
        sel = xn if all_logits else xn[rows - 1:rows]
        return ops.gemm_tc(sel, m.head, out32=torch.empty(sel.shape[0], c.vocab, dtype=torch.float32, device=self.dev))
