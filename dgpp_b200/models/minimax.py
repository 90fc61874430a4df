"""Block-sparse GQA + mixture-of-experts family (MiniMax-M3 style).

Every layer is grouped-query attention with per-head RMSNorm (1 + w) and partial rotary embedding on q / k, made
sparse by an index: each token stores one index key, each kv head owns one index query head; a row scores every block
of `sparse_block` tokens by the largest <index query, index key> among the block's visible tokens, always keeps its own
block and keeps the `sparse_topk` best blocks in all; the query heads of that kv head attend only to the tokens of
the kept blocks.  Feed-forward: dense or mixture-of-experts (sigmoid router with a selection bias, weights from the
uncorrected scores, normalised and scaled; one shared expert) with the activation
gate * sigmoid(alpha * gate) * (up + 1) after clamping gate above and up on both sides.  Norms are (1 + w) RMSNorms.

Oracle: ``MinimaxModel.forward_reference`` (dense masked attention in PyTorch); kernels: `rope_kv_write` (q / k norm,
rotary, FP8 KV append), `msa_index_prep` / `msa_index_select`, the paged decode attention in its block-selection form
(prefill rows included: every row carries its own block list), the MoE block, tensor-core linears.
(reference counterparts: src/models/minimax/layers.cpp MinimaxAttention::enqueue / MinimaxMlp, forward.cpp,
 reference.cpp select_blocks / attention / route / swiglu, src/kernels/minimax.cu.  The reference's NVFP4 KV cache and
 MXFP8 dense checkpoint format are not part of this build: KV is FP8 e4m3 per (token, head) scale, dense weights bf16
 or any format of this library's quantiser.)
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
class MinimaxConfig:
    layers: int = 4
    hidden: int = 512
    q_heads: int = 8
    kv_heads: int = 2               # = index heads
    head_dim: int = 128
    rotary_dim: int = 64
    rope_theta: float = 1e7
    eps: float = 1e-6
    index_dim: int = 128
    sparse_block: int = 64          # tokens per selectable block (= the KV page)
    sparse_topk: int = 4
    dense_ffn: int = 1024
    moe: Optional[MoEConfig] = None
    moe_layers: List[bool] = field(default_factory=list)      # per layer; empty: every layer when `moe` is set
    swiglu_alpha: float = 1.702
    swiglu_limit: float = 7.0
    vocab: int = 2048

    def is_moe(self, i: int) -> bool:
        return self.moe is not None and (not self.moe_layers or self.moe_layers[i])


@dataclass
class MinimaxLayer:
    in_norm: torch.Tensor            # [H] bf16, applied as 1 + w
    post_norm: torch.Tensor
    qkv: QuantLinear                 # [(hq + 2 hkv) d, H]
    q_norm: torch.Tensor             # [d]
    k_norm: torch.Tensor
    index: QuantLinear               # [(hkv + 1) di, H]: one index query head per kv head, then the index key
    index_q_norm: torch.Tensor       # [di]
    index_k_norm: torch.Tensor
    o: QuantLinear                   # [H, hq d]
    gate_up: Optional[QuantLinear] = None
    down: Optional[QuantLinear] = None
    moe: Optional[MoEWeights] = None


def select_blocks_reference(iq: torch.Tensor, ik: torch.Tensor, block: int, topk: int) -> torch.Tensor:
    """iq [T, ih, di], ik [T, di] fp32 (one request from position 0) -> bool [T, ih, nblocks]: the kept blocks of every
    (row, index head).  Block score = max over the block's visible tokens; the row's own block always wins; ties go to
    the lower block id."""
    T, ih, _ = iq.shape
    nb = (T + block - 1) // block
    s = torch.einsum("thd,sd->ths", iq, ik)                                   # [T, ih, T]
    t = torch.arange(T, device=iq.device)
    s = s.masked_fill((t.view(1, 1, T) > t.view(T, 1, 1)), float("-inf"))
    s = torch.nn.functional.pad(s, (0, nb * block - T), value=float("-inf")).view(T, ih, nb, block).amax(-1)
    own = (t // block).view(T, 1, 1).expand(T, ih, 1)
    s.scatter_(2, own, float("inf"))
    order = torch.argsort(-s, dim=-1, stable=True)[..., :topk]                # ties -> lower block id
    keep = torch.zeros(T, ih, nb, dtype=torch.bool, device=iq.device)
    keep.scatter_(2, order, True)
    return keep & (s > float("-inf"))                                          # blocks in the future are never kept


class MinimaxModel:
    def __init__(self, cfg: MinimaxConfig, embed, layers: List[MinimaxLayer], final_norm, head: QuantLinear, inv_freq):
        self.cfg, self.embed, self.layers, self.final_norm, self.head, self.inv_freq = cfg, embed, layers, final_norm, head, inv_freq

    @staticmethod
    def random_init(cfg: MinimaxConfig, device, seed: int = 0, std: float = 0.05, fmt: str = "bf16") -> "MinimaxModel":
        g = torch.Generator(device=device)
        g.manual_seed(seed)
        c, H, d, di = cfg, cfg.hidden, cfg.head_dim, cfg.index_dim
        rnd = lambda *s: torch.randn(*s, device=device, dtype=torch.float32, generator=g)
        lin = lambda n, k: quantize(rnd(n, k) * std, fmt if (k % 256 == 0 or fmt == "bf16") else "bf16")
        nw = lambda n: (0.1 * rnd(n)).to(BF)                                   # used as 1 + w
        layers = []
        for i in range(c.layers):
            L = MinimaxLayer(nw(H), nw(H), lin((c.q_heads + 2 * c.kv_heads) * d, H), nw(d), nw(d),
                             quantize(rnd((c.kv_heads + 1) * di, H) * std * 2, "bf16"), nw(di), nw(di), lin(H, c.q_heads * d))
            if c.is_moe(i):
                mc = c.moe
                assert mc.hidden == H and mc.swiglu_alpha == c.swiglu_alpha and mc.swiglu_limit == c.swiglu_limit
                L.moe = MoEWeights.random_init(mc, device, seed=seed * 1000 + i, std=std)
            else:
                L.gate_up, L.down = lin(2 * c.dense_ffn, H), lin(H, c.dense_ffn)
            layers.append(L)
        inv, _ = ref.rope_inv_freq(c.rotary_dim, c.rope_theta, device)
        return MinimaxModel(cfg, (rnd(c.vocab, H) * std * 4).to(BF), layers, nw(H), quantize(rnd(c.vocab, H) * std, "bf16"), inv)

    # ------------------------------------------------------------------ oracle
    def attention_reference(self, L: MinimaxLayer, xn: torch.Tensor, pos: torch.Tensor, return_keep: bool = False):
        c, d, di = self.cfg, self.cfg.head_dim, self.cfg.index_dim
        T = xn.shape[0]
        nq, nkv = c.q_heads * d, c.kv_heads * d
        qkv = ref.linear(xn, L.qkv).float()
        q = ref.apply_rope(ref.head_norm(qkv[:, :nq].view(T, c.q_heads, d), L.q_norm, c.eps, True), pos, self.inv_freq, c.rotary_dim)
        k = ref.apply_rope(ref.head_norm(qkv[:, nq:nq + nkv].view(T, c.kv_heads, d), L.k_norm, c.eps, True), pos, self.inv_freq,
                           c.rotary_dim)
        v = ref._r(qkv[:, nq + nkv:].view(T, c.kv_heads, d))
        iqk = ref.linear(xn, L.index).float().view(T, c.kv_heads + 1, di)
        iq = ref.apply_rope(ref.head_norm(iqk[:, :c.kv_heads], L.index_q_norm, c.eps, True), pos, self.inv_freq, c.rotary_dim)
        ik = ref.apply_rope(ref.head_norm(iqk[:, c.kv_heads:], L.index_k_norm, c.eps, True), pos, self.inv_freq, c.rotary_dim)[:, 0]
        keep = select_blocks_reference(iq, ik, c.sparse_block, c.sparse_topk)          # [T, hkv, nb]
        # the cache holds K / V as FP8 codes with one scale per (token, head)
        kq, ks = ref.quant_kv_fp8(k)
        vq, vs = ref.quant_kv_fp8(v)
        k = kq.view(torch.float8_e4m3fn).float() * ks.unsqueeze(-1)
        v = vq.view(torch.float8_e4m3fn).float() * vs.unsqueeze(-1)
        g = c.q_heads // c.kv_heads
        t = torch.arange(T, device=xn.device)
        allowed = keep[:, :, t // c.sparse_block] & (t.view(1, 1, T) <= t.view(T, 1, 1))      # [T, hkv, T]
        s = torch.einsum("qhd,khd->hqk", q, k.repeat_interleave(g, 1)) / math.sqrt(d)
        s = s.masked_fill(~allowed.permute(1, 0, 2).repeat_interleave(g, 0), float("-inf"))
        a = torch.einsum("hqk,khd->qhd", torch.softmax(s, -1), v.repeat_interleave(g, 1))
        out = ref.linear(ref.act(a.reshape(T, nq)), L.o)
        return (out, keep) if return_keep else out

    def ffn_reference(self, L: MinimaxLayer, xn: torch.Tensor) -> torch.Tensor:
        c = self.cfg
        if L.moe is not None:
            return moe_reference(xn, L.moe)
        return ref.linear(ref.swiglu(ref.linear(xn, L.gate_up), c.swiglu_limit, c.swiglu_alpha), L.down)

    def forward_reference(self, tokens: torch.Tensor) -> torch.Tensor:
        """fp32 logits [T, V] of one request from position 0."""
        c = self.cfg
        dev = self.embed.device
        T = tokens.numel()
        pos = torch.arange(T, device=dev)
        R = ref.embed_gather(tokens.to(dev), self.embed)
        delta = None
        for L in self.layers:
            xn, R = ref.rmsnorm(R, L.in_norm, c.eps, delta=delta, one_plus_w=True)
            delta = self.attention_reference(L, xn, pos)
            xn, R = ref.rmsnorm(R, L.post_norm, c.eps, delta=delta, one_plus_w=True)
            delta = self.ffn_reference(L, xn)
        xn, _ = ref.rmsnorm(R, self.final_norm, c.eps, delta=delta, one_plus_w=True)
        return ref.linear(xn, self.head, out_fp32=True)


class _IndexCache:
    """Paged index keys of one layer, addressed through the KV cache's block table."""

    def __init__(self, blocks: int, page: int, di: int, device):
        self.k = torch.zeros(blocks, page, di, dtype=BF, device=device)


class MinimaxRunner(RowRunner):
    def __init__(self, model: MinimaxModel, max_rows: int, slots: int, max_seq_len: int, device):
        c = model.cfg
        self.m, self.c = model, c
        self._init_rows(slots, device, kv_layers=c.layers, kv_heads=c.kv_heads, q_heads=c.q_heads, head_dim=c.head_dim,
                        page=c.sparse_block, max_seq_len=max_seq_len, max_rows=max_rows)
        blocks = self.kv.layers[0].k.shape[0]
        self.index = [_IndexCache(blocks, c.sparse_block, c.index_dim, device) for _ in range(c.layers)]
        self.max_sel = (max_seq_len + c.sparse_block - 1) // c.sparse_block + 1
        pool = {}
        self.moe = {i: MoEBlock(L.moe, min(max_rows, 16), device, pool=pool) for i, L in enumerate(model.layers)
                    if L.moe is not None and L.moe.gu_q is not None}
        e = lambda *s: torch.empty(*s, dtype=BF, device=device)
        H, d = c.hidden, c.head_dim
        self.R, self.xn, self.y = e(max_rows, H), e(max_rows, H), e(max_rows, H)
        self.qkv = e(max_rows, (c.q_heads + 2 * c.kv_heads) * d)
        self.iqk = e(max_rows, (c.kv_heads + 1) * c.index_dim)
        self.attn = e(max_rows, c.q_heads * d)
        self.sel = torch.empty(max_rows, c.kv_heads, c.sparse_topk, dtype=torch.int32, device=device)
        self.idx_scores = torch.empty(max_rows, c.kv_heads, self.max_sel, dtype=torch.float32, device=device)
        self.gu = e(max_rows, 2 * c.dense_ffn)
        self.act = e(max_rows, c.dense_ffn)
        # a row reads at most sparse_topk blocks: a few chunks per (row, kv head) fill the machine at decode widths
        self.splits = 8
        self.scratch = (torch.empty(max_rows * c.q_heads * self.splits * 2, dtype=torch.float32, device=device),
                        torch.empty(max_rows * c.q_heads * self.splits * d, dtype=torch.float32, device=device))

    def _attention(self, i: int, L: MinimaxLayer, xn, positions, row_req, out) -> None:
        c, rows = self.c, xn.shape[0]
        qkv, iqk, attn, sel = self.qkv[:rows], self.iqk[:rows], self.attn[:rows], self.sel[:rows]
        cache, bt = self.kv.layers[i], self.kv.block_table
        ops.linear(xn, L.qkv, out=qkv)
        ops.linear(xn, L.index, out=iqk)
        ops.rope_kv_write(qkv, positions, row_req, bt, self.m.inv_freq, cache, c.q_heads, c.kv_heads, c.head_dim,
                          rot_dim=c.rotary_dim, q_norm_w=L.q_norm, k_norm_w=L.k_norm, eps=c.eps, norm_one_plus_w=True)
        ops.msa_index_prep(iqk, positions, row_req, bt, self.m.inv_freq, L.index_q_norm, L.index_k_norm, self.index[i].k,
                           c.kv_heads, c.index_dim, c.rotary_dim, c.eps, one_plus_w=True)
        ops.msa_index_select(iqk, self.index[i].k, bt, row_req, positions, c.kv_heads, c.index_dim, c.sparse_block,
                             c.sparse_topk, self.max_sel, out=sel, scores=self.idx_scores[:rows])
        fn = ops.attn_decode_tc if (self.tc_attn and rows <= 32 and c.sparse_block % 16 == 0) else ops.attn_decode
        fn(qkv, qkv.stride(0), cache, bt, row_req, positions, c.q_heads, c.kv_heads, c.head_dim, self.att_scale,
           splits=self.splits, scratch=self.scratch, out=attn, sel=sel, sel_block=c.sparse_block)
        ops.linear(attn, L.o, out=out)

    def _ffn(self, i: int, L: MinimaxLayer, xn, out) -> None:
        c, rows = self.c, xn.shape[0]
        if L.moe is None:
            gu = ops.linear(xn, L.gate_up, out=self.gu[:rows])
            ops.linear(ops.swiglu(gu, out=self.act[:rows], limit=c.swiglu_limit, alpha=c.swiglu_alpha), L.down, out=out)
            return
        blk = self.moe.get(i)
        if blk is not None and rows <= blk.max_rows:
            blk.forward(xn, out)
        elif blk is not None:
            out.copy_(blk.forward_gathered(xn))
        else:
            out.copy_(moe_reference(xn, L.moe))

    @torch.no_grad()
    def forward(self, tokens, positions, row_req, chunk_slot=None, all_logits=True, pos0=None, extra=None):
        m, c = self.m, self.c
        rows = tokens.shape[0]
        R, xn, y = self.R[:rows], self.xn[:rows], self.y[:rows]
        ops.embed_gather(tokens, m.embed, out=R)
        delta = None
        for i, L in enumerate(m.layers):
            ops.rmsnorm(R, L.in_norm, c.eps, delta=delta, out=xn, one_plus_w=True)
            self._attention(i, L, xn, positions, row_req, y)
            ops.rmsnorm(R, L.post_norm, c.eps, delta=y, out=xn, one_plus_w=True)
            self._ffn(i, L, xn, y)
            delta = y
        ops.rmsnorm(R, m.final_norm, c.eps, delta=delta, out=xn, one_plus_w=True)
        sel = xn if all_logits else xn[rows - 1:rows]
        return ops.gemm_tc(sel, m.head, out32=torch.empty(sel.shape[0], c.vocab, dtype=torch.float32, device=self.dev))
