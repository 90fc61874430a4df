"""Looped transformer on the unit hypersphere (Dory style): the same stack of layers runs `loops` times over the hidden
state, every sub-block's output moves the state along the sphere instead of being added to it.

    x_0      = justnorm(embed[token])
    per loop, per layer:
        a    = W_o attention(rope(W_qkv x))            x = justnorm(x^ + |alpha_a s_a| (a^ - x^))     (^ = unit norm)
        h    = W_down swiglu(W_gate_up x)              x = justnorm(x^ + |alpha_m s_m| (h^ - x^))
    logits   = logit_scale * W_head x

Weights are shared by the loops; the KV cache is not (loop r of layer l owns cache layer r * layers + l).  Single GPU
only, like the family it follows.  Oracle: ``DoryModel.forward_reference``; kernels: `justnorm`, `slerp_alpha` (fp64
row sums), tensor-core linears, rotary + FP8 KV append, tcgen05 attention.
(reference counterparts: src/models/dory/forward.cpp, layers.cpp, src/kernels/dory_norm.cu, dory_attn.cu, dory_head.cu.)
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import List

import torch

from ..ops import core as ops
from ..ops import reference as ref
from ..quant.formats import QuantLinear, quantize
from .rows import RowRunner

BF = torch.bfloat16


@dataclass
class DoryConfig:
    layers: int = 2
    loops: int = 3
    hidden: int = 512
    q_heads: int = 4
    kv_heads: int = 2
    head_dim: int = 128
    ffn: int = 1024
    vocab: int = 2048
    rope_theta: float = 1e4
    eps: float = 1e-6
    s_att: float = 0.05          # step scales of the two residual kinds
    s_mlp: float = 0.05
    logit_scale: float = 8.0
    page: int = 64


@dataclass
class DoryLayer:
    qkv: QuantLinear
    o: QuantLinear
    gate_up: QuantLinear
    down: QuantLinear
    alpha_a: torch.Tensor        # [H] bf16: per-channel step size
    alpha_m: torch.Tensor


class DoryModel:
    def __init__(self, cfg: DoryConfig, embed, layers: List[DoryLayer], head: QuantLinear, inv_freq):
        self.cfg, self.embed, self.layers, self.head, self.inv_freq = cfg, embed, layers, head, inv_freq

    @staticmethod
    def random_init(cfg: DoryConfig, device, seed: int = 0, std: float = 0.05, fmt: str = "bf16") -> "DoryModel":
        g = torch.Generator(device=device)
        g.manual_seed(seed)
        c, H, d = cfg, cfg.hidden, cfg.head_dim
        rnd = lambda *s: torch.randn(*s, device=device, dtype=torch.float32, generator=g)
        lin = lambda n, k: quantize(rnd(n, k) * std, fmt)
        layers = [DoryLayer(lin((c.q_heads + 2 * c.kv_heads) * d, H), lin(H, c.q_heads * d), lin(2 * c.ffn, H), lin(H, c.ffn),
                            ((1 + 0.2 * rnd(H)) * 4).to(BF), ((1 + 0.2 * rnd(H)) * 4).to(BF)) for _ in range(c.layers)]
        inv, _ = ref.rope_inv_freq(d, c.rope_theta, device)
        return DoryModel(cfg, (rnd(c.vocab, H) * std).to(BF), layers, quantize(rnd(c.vocab, H) * std, "bf16"), inv)

    def forward_reference(self, tokens: torch.Tensor) -> torch.Tensor:
        """fp32 logits [T, V] of one request from position 0."""
        c, d = self.cfg, self.cfg.head_dim
        T = tokens.numel()
        pos = torch.arange(T, device=self.embed.device)
        nq, nkv = c.q_heads * d, c.kv_heads * d
        x = ref.justnorm(ref.embed_gather(tokens.to(self.embed.device), self.embed), c.eps)
        for _ in range(c.loops):
            for L in self.layers:
                qkv = ref.linear(x, L.qkv).float()
                q = ref.apply_rope(qkv[:, :nq].view(T, c.q_heads, d), pos, self.inv_freq, d)
                k = ref.apply_rope(qkv[:, nq:nq + nkv].view(T, c.kv_heads, d), pos, self.inv_freq, d)
                v = ref._r(qkv[:, nq + nkv:].view(T, c.kv_heads, d))
                a = ref.attention(q, k, v, 1.0 / math.sqrt(d), causal_offset=0)
                x = ref.slerp_alpha(x, ref.linear(ref.act(a.reshape(T, nq)), L.o), L.alpha_a, c.s_att, c.eps)
                h = ref.linear(ref.swiglu(ref.linear(x, L.gate_up)), L.down)
                x = ref.slerp_alpha(x, h, L.alpha_m, c.s_mlp, c.eps)
        return ref.linear(x, self.head, out_fp32=True) * c.logit_scale


class DoryRunner(RowRunner):
    def __init__(self, model: DoryModel, max_rows: int, slots: int, max_seq_len: int, device):
        c = model.cfg
        self.m, self.c = model, c
        self._init_rows(slots, device, kv_layers=c.loops * c.layers, kv_heads=c.kv_heads, q_heads=c.q_heads,
                        head_dim=c.head_dim, page=c.page, max_seq_len=max_seq_len, max_rows=max_rows)
        e = lambda *s: torch.empty(*s, dtype=BF, device=device)
        self.qkv = e(max_rows, (c.q_heads + 2 * c.kv_heads) * c.head_dim)
        self.attn, self.h = e(max_rows, c.q_heads * c.head_dim), e(max_rows, c.hidden)

    @torch.no_grad()
    def forward(self, tokens, positions, row_req, chunk_slot=None, all_logits=True, pos0=None, extra=None):
        m, c = self.m, self.c
        rows = tokens.shape[0]
        x = ops.justnorm(ops.embed_gather(tokens, m.embed, out=self.h[:rows]), c.eps)
        qkv, attn, h = self.qkv[:rows], self.attn[:rows], self.h[:rows]
        for r in range(c.loops):
            for l, L in enumerate(m.layers):
                ops.linear(x, L.qkv, out=qkv)
                self._attention_rows(r * c.layers + l, qkv, positions, row_req, m.inv_freq, chunk_slot, pos0, attn)
                x = ops.slerp_alpha(x, ops.linear(attn, L.o, out=h), L.alpha_a, c.s_att, c.eps)
                ops.linear(ops.swiglu(ops.linear(x, L.gate_up)), L.down, out=h)
                x = ops.slerp_alpha(x, h, L.alpha_m, c.s_mlp, c.eps)
        sel = x if all_logits else x[rows - 1:rows]
        logits = ops.gemm_tc(sel, m.head, out32=torch.empty(sel.shape[0], c.vocab, dtype=torch.float32, device=self.dev))
        return logits.mul_(c.logit_scale)
