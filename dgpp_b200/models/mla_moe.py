"""MLA + MoE decoder family (DeepSeek-V3 / GLM-DSA style): multi-head latent attention with a low-rank query path,
optional lightning-indexer sparse attention, dense or mixture-of-experts FFN.

Per layer (token x, RMSNorm pre-norms, residual stream in bf16):
    c_q   = norm(W_qa x)                      [q_lora]
    q     = W_qb c_q                          [heads, nope + rope]      (rope part rotated)
    c_kv  = norm((W_kva x)[:dc]),  k_r = rope((W_kva x)[dc:])            cache row = [c_kv | k_r]  (dc + dr per token)
    k_h   = [W_uk_h c_kv | k_r],  v_h = W_uv_h c_kv                      (never materialised by the kernel path)
    a_h   = softmax(q_h . k_h / sqrt(nope + rope)) v_h ;  out = W_o [a_1 .. a_H]
The kernel path runs the ABSORBED form: q_abs_h = W_uk_h^T q_nope_h (so the score is q_abs . c + q_r . k_r against the
shared cache row) and a_h = W_uv_h (sum_t p_t c_t); the oracle below runs the plain form, so agreement checks the
absorption as well as the kernels.  With the sparse index, every query row keeps the top-k cached positions by
sum_i w_i relu(q_idx_i . k_idx_t) (k_idx cached per token) and attends only to them.
(reference counterparts: src/models/glm_dsa/model.cpp, src/models/dsa_layer.cu, dsa_reference.cpp, the MoE layers of
 src/models/glm/moe_layer.cpp; kernels src/kernels/dsa.cu.)
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import List, Optional

import torch

from ..ops import core as ops
from ..ops import reference as ref
from ..quant.formats import QuantLinear, quantize
from .moe import MoEBlock, MoEConfig, MoEWeights, moe_reference

BF = torch.bfloat16


@dataclass
class MlaMoeConfig:
    layers: int = 4
    hidden: int = 1024
    heads: int = 8
    q_lora: int = 256
    kv_lora: int = 128           # dc
    nope: int = 64
    rope: int = 32               # dr
    v_dim: int = 64
    ffn: int = 2048              # dense layers
    dense_layers: int = 1        # the first layers use a dense FFN, the rest the MoE
    vocab: int = 4096
    eps: float = 1e-6
    rope_theta: float = 1e4
    # YaRN context extension of the rotary part (factor 1 = plain RoPE): frequencies whose wavelength exceeds the
    # original context are interpolated by `yarn_factor`, fast ones are kept, a linear ramp in between; the softmax
    # scale is multiplied by (0.1 ln(factor) + 1)^2
    yarn_factor: float = 1.0
    yarn_orig_ctx: int = 4096
    yarn_beta_fast: float = 32.0
    yarn_beta_slow: float = 1.0
    page: int = 64
    moe: Optional[MoEConfig] = None
    # sparse index (0 heads = dense attention everywhere)
    index_heads: int = 0
    index_dim: int = 64
    index_topk: int = 64
    index_key_fp8: bool = False  # index keys cached as e4m3 with one scale per token (index_dim 128, tensor-core kernel)


@dataclass
class MlaLayer:
    in_norm: torch.Tensor
    post_norm: torch.Tensor
    q_a: QuantLinear             # [q_lora, H]
    q_a_norm: torch.Tensor
    q_b: QuantLinear             # [heads * (nope + rope), q_lora]
    kv_a: QuantLinear            # [dc + dr, H]
    kv_a_norm: torch.Tensor
    w_uk: torch.Tensor           # [heads, nope, dc] bf16
    w_uv: torch.Tensor           # [heads, v, dc] bf16
    o: QuantLinear               # [H, heads * v]
    gate_up: Optional[QuantLinear] = None
    down: Optional[QuantLinear] = None
    moe: Optional[MoEWeights] = None
    idx_q: Optional[QuantLinear] = None   # [hi * di, H]
    idx_k: Optional[QuantLinear] = None   # [di, H]
    idx_w: Optional[QuantLinear] = None   # [hi, H]


def _rope(x: torch.Tensor, pos: torch.Tensor, inv_freq: torch.Tensor) -> torch.Tensor:
    """x [..., T?, d] with leading token axis 0: rotate-half convention on the last axis.  fp32 in / out."""
    ang = pos.float().unsqueeze(-1) * inv_freq                     # [T, d/2]
    while ang.dim() < x.dim():
        ang = ang.unsqueeze(1)
    c, s = torch.cos(ang), torch.sin(ang)
    h = x.shape[-1] // 2
    a, b = x[..., :h], x[..., h:]
    return torch.cat([a * c - b * s, b * c + a * s], -1)


def yarn_inv_freq(dim: int, theta: float, factor: float, orig_ctx: int, beta_fast: float = 32.0, beta_slow: float = 1.0,
                  device=None) -> torch.Tensor:
    """Rotary inverse frequencies [dim / 2] under YaRN scaling (factor <= 1: the plain table)."""
    extra = 1.0 / (theta ** (torch.arange(0, dim, 2, device=device).float() / dim))
    if factor <= 1.0:
        return extra
    corr = lambda rot: dim * math.log(orig_ctx / (rot * 2 * math.pi)) / (2 * math.log(theta))
    low, high = max(math.floor(corr(beta_fast)), 0), min(math.ceil(corr(beta_slow)), dim // 2 - 1)
    ramp = ((torch.arange(dim // 2, device=device).float() - low) / max(high - low, 1e-3)).clamp(0, 1)
    return extra / factor * ramp + extra * (1 - ramp)


def softmax_scale(c) -> float:
    """1 / sqrt(nope + rope), times the YaRN magnitude correction when the config extends the context."""
    f = float(getattr(c, "yarn_factor", 1.0))
    m = 0.1 * math.log(f) + 1.0 if f > 1.0 else 1.0
    return m * m / math.sqrt(c.nope + c.rope)


def mla_attention_reference(c, inv_freq: torch.Tensor, L: "MlaLayer", xn: torch.Tensor, pos: torch.Tensor) -> torch.Tensor:
    """Plain (non-absorbed) latent attention of consecutive tokens of one request from position 0, with the sparse
    index when the layer has one.  c: any config with heads / q_lora / kv_lora / nope / rope / v_dim / index_* / eps.
    xn [T, H] bf16 normed rows -> o [T, H] bf16 (after the output projection)."""
    T = xn.shape[0]
    scale = softmax_scale(c)
    cq = ref.rmsnorm(ref.linear(xn, L.q_a), L.q_a_norm, c.eps)[0]
    q = ref.linear(cq, L.q_b).float().view(T, c.heads, c.nope + c.rope)
    q_n, q_r = q[..., :c.nope], ref._r(_rope(q[..., c.nope:], pos, inv_freq))
    kv = ref.linear(xn, L.kv_a)
    ckv = ref.rmsnorm(kv[:, :c.kv_lora].contiguous(), L.kv_a_norm, c.eps)[0].float()         # bf16 values
    k_r = ref._r(_rope(kv[:, c.kv_lora:].float(), pos, inv_freq))                        # [T, dr]
    k_n = torch.einsum("hnd,td->thn", L.w_uk.float(), ckv)                                    # [T, heads, nope]
    v = torch.einsum("hvd,td->thv", L.w_uv.float(), ckv)                                      # [T, heads, v]
    s = (torch.einsum("qhn,khn->hqk", q_n, k_n) + torch.einsum("qhr,kr->hqk", q_r, k_r)) * scale
    mask = pos.unsqueeze(0) > pos.unsqueeze(1)                                                # [q, k]
    if L.idx_q is not None:
        qi = ref.linear(xn, L.idx_q).float().view(T, c.index_heads, c.index_dim)
        ki = ref.linear(xn, L.idx_k).float()                                                  # [T, di]
        if getattr(c, "index_key_fp8", False):             # the cache holds e4m3(k / scale), scale = amax / 448 per token
            sc = (ki.abs().amax(-1, keepdim=True) / 448.0).clamp_min(1e-30)
            sc = torch.where(ki.abs().amax(-1, keepdim=True) > 0, sc, torch.ones_like(sc))
            ki = (ki / sc).to(torch.float8_e4m3fn).float() * sc
        wi = ref.linear(xn, L.idx_w).float()                                                  # [T, hi]
        sc = (torch.relu(torch.einsum("qhd,kd->qhk", qi, ki)) * wi.unsqueeze(-1)).sum(1)      # [q, k]
        sc = sc.masked_fill(mask, float("-inf"))
        keep = torch.zeros_like(mask)
        for t in range(T):
            n = t + 1
            if n <= c.index_topk:
                keep[t, :n] = True
            else:
                order = torch.argsort(-sc[t, :n], stable=True)[:c.index_topk]                 # ties -> lower position
                keep[t, order] = True
        mask = mask | ~keep
    p = torch.softmax(s.masked_fill(mask.unsqueeze(0), float("-inf")), -1)
    a = ref._r(torch.einsum("hqk,khv->qhv", p, v)).reshape(T, c.heads * c.v_dim)
    o = ref.linear(ref.act(a), L.o)
    return o


class MlaMoeModel:
    def __init__(self, cfg: MlaMoeConfig, embed, layers: List[MlaLayer], final_norm, head: QuantLinear, inv_freq):
        self.cfg, self.embed, self.layers, self.final_norm, self.head, self.inv_freq = cfg, embed, layers, final_norm, head, inv_freq

    @staticmethod
    def random_init(cfg: MlaMoeConfig, device, seed: int = 0, std: float = 0.05, fmt: str = "bf16", ep_rank: int = 0,
                    ep_size: int = 1) -> "MlaMoeModel":
        """ep_size > 1 (expert parallelism): every rank draws the same model and keeps its contiguous block of every MoE
        layer's experts (plus a copy of the shared expert, which runs on the rank's own rows); everything else is replicated."""
        g = torch.Generator(device=device)
        g.manual_seed(seed)
        rnd = lambda n, k: torch.randn(n, k, device=device, dtype=torch.float32, generator=g) * std
        lin = lambda n, k: quantize(rnd(n, k), fmt if (k % 256 == 0 or fmt == "bf16") else "bf16")
        ones = lambda n: torch.ones(n, device=device, dtype=BF)
        H, c = cfg.hidden, cfg
        layers = []
        for i in range(cfg.layers):
            L = MlaLayer(ones(H), ones(H), lin(c.q_lora, H), ones(c.q_lora), lin(c.heads * (c.nope + c.rope), c.q_lora),
                         lin(c.kv_lora + c.rope, H), ones(c.kv_lora),
                         (torch.randn(c.heads, c.nope, c.kv_lora, device=device, generator=g) * std * 2).to(BF),
                         (torch.randn(c.heads, c.v_dim, c.kv_lora, device=device, generator=g) * std * 2).to(BF),
                         lin(H, c.heads * c.v_dim))
            if cfg.moe is not None and i >= cfg.dense_layers:
                L.moe = MoEWeights.random_init(cfg.moe, device, seed=seed * 1000 + i, std=std, ep_rank=ep_rank, ep_size=ep_size,
                                               shared_everywhere=ep_size > 1)
            else:
                L.gate_up, L.down = lin(2 * c.ffn, H), lin(H, c.ffn)
            if cfg.index_heads:
                L.idx_q = quantize(rnd(c.index_heads * c.index_dim, H) * 4, fmt)
                L.idx_k = quantize(rnd(c.index_dim, H) * 4, "bf16")
                L.idx_w = quantize(rnd(c.index_heads, H), "bf16")
            layers.append(L)
        embed = (torch.randn(cfg.vocab, H, device=device, generator=g) * std).to(BF)
        inv = yarn_inv_freq(cfg.rope, cfg.rope_theta, cfg.yarn_factor, cfg.yarn_orig_ctx, cfg.yarn_beta_fast,
                            cfg.yarn_beta_slow, device)
        return MlaMoeModel(cfg, embed, layers, ones(H), quantize(rnd(cfg.vocab, H), "bf16"), inv)

    # ------------------------------------------------------------------ oracle (plain, non-absorbed attention)
    def forward_reference(self, tokens: torch.Tensor) -> torch.Tensor:
        """Logits [T, V] of one request from position 0 (PyTorch, fp32 accumulation, bf16 rounding at the points the
        kernel path rounds: projections, cache rows, attention output, FFN output)."""
        c = self.cfg
        T = tokens.numel()
        dev = self.embed.device
        pos = torch.arange(T, device=dev)
        x = ref.embed_gather(tokens.to(dev), self.embed)
        delta = None
        scale = 1.0 / math.sqrt(c.nope + c.rope)
        for L in self.layers:
            xn, x = ref.rmsnorm(x, L.in_norm, c.eps, delta)
            o = mla_attention_reference(c, self.inv_freq, L, xn, pos)
            xn, x = ref.rmsnorm(x, L.post_norm, c.eps, o)
            if L.moe is not None:
                delta = moe_reference(xn, L.moe)
            else:
                delta = ref.linear(ref.swiglu(ref.linear(xn, L.gate_up)), L.down)
        xn, x = ref.rmsnorm(x, self.final_norm, c.eps, delta)
        return ref.linear(xn, self.head, out_fp32=True)


class MlaCaches:
    """Paged latent cache (+ index-key cache) of the MLA layers of a model and the absorbed-attention launch sequence
    of one layer.  Shared by the families that contain MLA layers."""

    def __init__(self, c, layers: int, indexed: List[bool], max_rows: int, slots: int, max_seq_len: int, device,
                 shared_tail_blocks: int = 0):
        """shared_tail_blocks > 0: memory for ONE full-length request plus that many private blocks for each further
        slot; `share_prefix` then lets the other slots read the first slot's prefix (requests that continue a common
        long prefix, when independent full-length caches would not fit)."""
        self.c, self.dev = c, device
        self.page = c.page
        self.max_blocks = (max_seq_len + c.page - 1) // c.page + 1
        self.tail_blocks = shared_tail_blocks
        nblocks = (self.max_blocks + (slots - 1) * shared_tail_blocks if shared_tail_blocks else slots * self.max_blocks) + 1
        self.max_ctx = self.max_blocks * c.page
        self.latent = [torch.zeros(nblocks, c.page, c.kv_lora + c.rope, dtype=BF, device=device) for _ in range(layers)]
        self.key_fp8 = bool(getattr(c, "index_key_fp8", False))
        self.kidx = [torch.zeros(nblocks, c.page, c.index_dim, dtype=torch.uint8 if self.key_fp8 else BF, device=device)
                     if ix else None for ix in indexed]
        self.kscale = [torch.ones(nblocks, c.page, dtype=torch.float32, device=device) if ix and self.key_fp8 else None
                       for ix in indexed]
        # static block table: slot s owns blocks [1 + s * max_blocks, 1 + (s + 1) * max_blocks)
        if shared_tail_blocks:
            self.block_table = torch.zeros(slots, self.max_blocks, dtype=torch.int32, device=device)
            self.block_table[0] = 1 + torch.arange(self.max_blocks, device=device, dtype=torch.int32)
        else:
            self.block_table = (1 + torch.arange(slots * self.max_blocks, device=device, dtype=torch.int32)
                                ).view(slots, self.max_blocks).contiguous()
        self.scale = softmax_scale(c)
        self.scores = torch.empty(max_rows, self.max_ctx, dtype=torch.float32, device=device) if any(indexed) else None
        self.dq = ops.DecodeQuant(device)

    def share_prefix(self, dst: int, tokens: int) -> None:
        """Slot `dst` reads the first `tokens` positions (a multiple of the page) from slot 0's blocks and appends into
        its own tail blocks."""
        assert self.tail_blocks and dst > 0 and tokens % self.page == 0
        n = tokens // self.page
        assert n + self.tail_blocks <= self.max_blocks
        first = 1 + self.max_blocks + (dst - 1) * self.tail_blocks
        row = torch.zeros(self.max_blocks, dtype=torch.int32, device=self.dev)
        row[:n] = self.block_table[0, :n]
        row[n:n + self.tail_blocks] = first + torch.arange(self.tail_blocks, device=self.dev, dtype=torch.int32)
        self.block_table[dst].copy_(row)

    def clone_prefix(self, dst: int, tokens: int) -> None:
        """Copies the cache rows of slot 0's first `tokens` positions into slot `dst`'s own blocks."""
        assert not self.tail_blocks
        n = (tokens + self.page - 1) // self.page
        src, to = self.block_table[0, :n].long(), self.block_table[dst, :n].long()
        for cache in list(self.latent) + [k for k in self.kidx if k is not None] + [k for k in self.kscale if k is not None]:
            cache.index_copy_(0, to, cache.index_select(0, src))

    def _append(self, cache: torch.Tensor, rows: torch.Tensor, row_req: torch.Tensor, positions: torch.Tensor) -> None:
        blk = self.block_table[row_req.long(), (positions // self.page).long()].long()
        cache[blk, (positions % self.page).long()] = rows

    def attention(self, j: int, L: MlaLayer, inv_freq: torch.Tensor, xn: torch.Tensor, positions: torch.Tensor,
                  row_req: torch.Tensor, select: bool, out: torch.Tensor, xa=None, fp4: bool = True) -> torch.Tensor:
        """xn [rows, H] normed rows of MLA layer j -> out [rows, H] (after the output projection).  Appends the rows'
        latent (and index key) to the cache first; every row attends up to its own position.  xa: the NVFP4 terms of xn
        when the caller's norm kernel produced them (decode widths): the projections then run block-scaled."""
        c, dq = self.c, self.dq
        rows = xn.shape[0]
        fast = fp4 and dq.usable(rows, L.q_a, L.q_b, L.kv_a, L.o)
        if fast:
            xa = xa if xa is not None else dq.plain(xn, "h")
            cqa = dq.norm(ops.gemm_fp4(xa, L.q_a), L.q_a_norm, c.eps, tag="q")
            q = ops.gemm_fp4(cqa, L.q_b).view(rows, c.heads, c.nope + c.rope)
            kv = ops.gemm_fp4(xa, L.kv_a)
        else:
            cq = ops.rmsnorm(ops.linear(xn, L.q_a), L.q_a_norm, c.eps)
            q = ops.linear(cq, L.q_b).view(rows, c.heads, c.nope + c.rope)
            kv = ops.linear(xn, L.kv_a)
        # latent norm + rotary key -> cache slot; key up-projection folded into the query, rotary part appended
        ops.mla_kv_prep(kv, L.kv_a_norm, c.eps, inv_freq, positions, row_req, self.block_table, self.latent[j],
                        c.kv_lora, c.rope)
        q_full = ops.mla_q_absorb(q, L.w_uk, inv_freq, positions, c.kv_lora, c.rope)
        sel = None
        if L.idx_q is not None and self.key_fp8:
            ops.dsa_key_append_fp8(ops.linear(xn, L.idx_k), positions, row_req, self.block_table, self.kidx[j], self.kscale[j])
        elif L.idx_q is not None:
            self._append(self.kidx[j], ops.linear(xn, L.idx_k), row_req, positions)
        if L.idx_q is not None and select:
            qi = (ops.gemm_fp4(xa, L.idx_q) if fast and dq.usable(rows, L.idx_q) else ops.linear(xn, L.idx_q)
                  ).view(rows, c.index_heads, c.index_dim)
            wi = ops.linear(xn, L.idx_w).float().contiguous()
            sc = ops.dsa_index(qi, wi, self.kidx[j], self.block_table, row_req, positions, self.max_ctx,
                               scores=self.scores[:rows], k_scale=self.kscale[j])
            sel = ops.topk_select(sc, positions, c.index_topk)
        # decode rows: enough (row, head group, context split) CTAs to cover the SMs; a split beyond a short context
        # writes an empty partial, so the count depends on the batch width only (a captured pass stays valid)
        splits = max(1, min(64, -(-148 // (rows * -(-c.heads // 32))))) if rows <= 16 else 1
        lat = ops.mla_decode(q_full, self.latent[j], self.block_table, row_req, positions, self.scale, c.kv_lora,
                             c.rope, sel=sel, splits=splits)
        a = ops.mla_v_up(lat, L.w_uv)
        if fast:
            return ops.gemm_fp4(dq.plain(a, "a"), L.o, out=out)
        return ops.linear(a, L.o, out=out)


class MlaMoeRunner:
    """Kernel execution: latent cache + index-key cache in pages, absorbed MLA decode kernel (dense or sparse), MoE
    block, tensor-core linears.  Rows may be a prefill chunk of one request or one decode token per request."""

    def __init__(self, model: MlaMoeModel, max_rows: int, slots: int, max_seq_len: int, device, shared_tail_blocks: int = 0):
        c = model.cfg
        self.m, self.c, self.dev, self.max_rows = model, c, device, max_rows
        self.att = MlaCaches(c, len(model.layers), [L.idx_q is not None for L in model.layers], max_rows, slots,
                             max_seq_len, device, shared_tail_blocks)
        self.page, self.max_blocks, self.max_ctx = self.att.page, self.att.max_blocks, self.att.max_ctx
        self.latent, self.kidx, self.block_table = self.att.latent, self.att.kidx, self.att.block_table
        self.lengths = [0] * slots
        # expert parallelism: a model whose MoE layers hold a block of the experts runs them through the token-sharded
        # all-to-all (this rank's rows go to the experts' owners and come back); every rank then calls the model in
        # lockstep, each with its own rows.  One communicator and one set of tile buffers serve all layers.
        self.ep, self.ep_small = {}, {}
        first = next((L.moe for L in model.layers if L.moe is not None), None)
        if first is not None and (first.e_end or c.moe.experts) - first.e_begin < c.moe.experts:
            from ..parallel.ep import EpMoE
            comm, pool, pool_small = None, {}, {}
            for i, L in enumerate(model.layers):
                if L.moe is not None:
                    self.ep[i] = EpMoE(L.moe, max_rows, device, comm=comm, pool=pool)
                    comm = comm or (self.ep[i].comm, self.ep[i].world, self.ep[i].rank, self.ep[i]._blob)
                    # decode widths get their own small tile lists (the prefill-sized ones cost a decode step their grid)
                    self.ep_small[i] = EpMoE(L.moe, 16, device, comm=comm, pool=pool_small) if max_rows > 16 else self.ep[i]
        self.moe = {i: MoEBlock(L.moe, min(max_rows, 16), device) for i, L in enumerate(model.layers)
                    if L.moe is not None and L.moe.gu_q is not None and not self.ep}
        self.decode_fp4 = True      # decode-width passes: NVFP4 linears on the block-scaled path (three-term activations)
        self.use_graphs, self._graphs, self._static = True, {}, {}
        self.pdl_graphs = True      # programmatic-dependent-launch edges between this library's kernels in captured passes

    def reset(self, slot: int) -> None:
        self.lengths[slot] = 0

    def _state_tensors(self):
        return []          # the latent / index-key cache writes of a pass are idempotent

    @torch.no_grad()
    def forward(self, tokens: torch.Tensor, positions: torch.Tensor, row_req: torch.Tensor,
                all_logits: bool = True, select: bool = True) -> torch.Tensor:
        """int32 [rows] device tensors -> fp32 logits [rows, V] (all_logits=False: of the last row only, [1, V]).
        select=False (indexed models): the caller knows that no row's context exceeds the selection size, so every
        token is selected and the dense attention kernel runs; the index keys are still appended."""
        m, c = self.m, self.c
        rows = tokens.shape[0]
        x = torch.empty(rows, c.hidden, dtype=BF, device=self.dev)
        xn, delta = torch.empty_like(x), torch.empty_like(x)
        ops.embed_gather(tokens, m.embed, out=x)
        have = False
        dq = self.att.dq
        for i, L in enumerate(m.layers):
            fast = self.decode_fp4 and dq.usable(rows, L.q_a, L.q_b, L.kv_a, L.o)
            xa = None
            if fast:      # norm + residual add + NVFP4 terms in one kernel; xn is still needed (bf16 linears, router)
                xa = dq.norm(x, L.in_norm, c.eps, delta=delta if have else None, x_out=xn, tag="h")
            else:
                ops.rmsnorm(x, L.in_norm, c.eps, delta=delta if have else None, out=xn)
            self.att.attention(i, L, m.inv_freq, xn, positions, row_req, select, delta, xa=xa, fp4=fast)
            if fast:
                xa = dq.norm(x, L.post_norm, c.eps, delta=delta, x_out=xn, tag="h")
            else:
                ops.rmsnorm(x, L.post_norm, c.eps, delta=delta, out=xn)
            have = True
            if L.moe is not None and i in self.ep:
                (self.ep_small[i] if rows <= 16 else self.ep[i]).forward(xn, out=delta)
            elif L.moe is not None:
                blk = self.moe.get(i)
                if blk is not None and rows <= blk.max_rows:
                    blk.forward(xn, delta, xa=xa if (fast and blk.bn == dq.ROWS and blk.terms == dq.TERMS) else None)
                elif blk is not None:
                    delta.copy_(blk.forward_gathered(xn))
                else:
                    delta.copy_(moe_reference(xn, L.moe))
            elif fast and dq.usable(rows, L.gate_up, L.down):
                ops.gemm_fp4(dq.swiglu(ops.gemm_fp4(xa, L.gate_up), tag="f"), L.down, out=delta)
            else:
                ops.linear(ops.swiglu(ops.linear(xn, L.gate_up)), L.down, out=delta)
        ops.rmsnorm(x, m.final_norm, c.eps, delta=delta, out=xn)
        sel_rows = xn if all_logits else xn[rows - 1:rows]
        return ops.gemm_tc(sel_rows, m.head, out32=torch.empty(sel_rows.shape[0], c.vocab, dtype=torch.float32, device=self.dev))

    @torch.no_grad()
    def prefill(self, slot: int, tokens: List[int], chunk: int = 64) -> torch.Tensor:
        start = self.lengths[slot]
        assert start + len(tokens) <= self.max_ctx - self.page
        out = None
        for o in range(0, len(tokens), chunk):
            part = tokens[o:o + chunk]
            t = torch.tensor(part, dtype=torch.int32, device=self.dev)
            pos = torch.arange(start + o, start + o + len(part), dtype=torch.int32, device=self.dev)
            req = torch.full((len(part),), slot, dtype=torch.int32, device=self.dev)
            out = self.forward(t, pos, req, all_logits=False, select=start + o + len(part) > self.c.index_topk)
        self.lengths[slot] = start + len(tokens)
        return out

    def _decode_rows(self, slots: List[int], tokens: List[int], positions: List[int]) -> torch.Tensor:
        """One decode pass.  On a GPU the pass is captured once per batch width into a CUDA graph over static id /
        position / request tensors and replayed (a pass is hundreds of small launches; replay removes the host's
        launch cost from every step); `use_graphs = False` launches kernel by kernel."""
        b = len(slots)
        select = bool(self.c.index_heads) and max(positions) + 1 > self.c.index_topk
        host = torch.tensor([tokens, positions, slots], dtype=torch.int32)
        if not (self.use_graphs and torch.device(self.dev).type == "cuda"):
            d = host.to(self.dev)
            return self.forward(d[0], d[1], d[2], select=select)
        key = (b, select)
        st = self._static.get(key)
        if st is None:
            st = self._static[key] = torch.zeros(3, b, dtype=torch.int32, device=self.dev)
        st.copy_(host, non_blocking=True)
        g = self._graphs.get(key)
        if g is None:
            # warm-up outside capture (lazy kernel attributes, workspaces); state-carrying layers are advanced by it,
            # so their state is saved before and put back after: only replays move the model forward
            saved = [t.clone() for t in self._state_tensors()]
            side = torch.cuda.Stream()
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                self.forward(st[0], st[1], st[2], select=select)
            torch.cuda.current_stream().wait_stream(side)
            torch.cuda.synchronize()
            from ..engine.graph import capture_with_pdl
            graph, out, _ = capture_with_pdl(lambda: self.forward(st[0], st[1], st[2], select=select), self.pdl_graphs)
            for t, s0 in zip(self._state_tensors(), saved):
                t.copy_(s0)
            g = self._graphs[key] = (graph, out)
        graph, out = g
        graph.replay()
        return out

    @torch.no_grad()
    def decode(self, slots: List[int], tokens: List[int]) -> torch.Tensor:
        out = self._decode_rows(slots, tokens, [self.lengths[s] for s in slots])
        for s in slots:
            self.lengths[s] += 1
        return out
