"""Kernel-path execution of the dense decoder: one `DenseRunner` owns the static activation buffers
and issues the sm_100a kernels for a batch of rows (prefill chunk or decode batch).

Every buffer is allocated once, so a forward pass is a pure sequence of kernel launches on the
current stream: it can be captured into a CUDA graph as is (no allocation, no host sync).
Row-split projections (o_proj, down) are followed by the tensor-parallel reduction supplied by a
`Reducer` (``dgpp_b200.parallel``): the fused peer-memory kernel, or NCCL as the baseline.
(reference call stack being replaced: src/models/qwen/model35.cpp:2066-2399 run_rows.)
"""
from __future__ import annotations

import math
from typing import Optional

import torch

from ..models.dense import DenseModel
from ..ops import core as ops
from .kv_cache import PagedKV

BF = torch.bfloat16


class DenseRunner:
    def __init__(self, model: DenseModel, kv: PagedKV, max_rows: int, reducer=None, decode_splits: int = 8):
        self.m, self.kv, self.max_rows, self.reducer = model, kv, max_rows, reducer
        c = model.cfg
        dev = model.embed.device
        d = c.head_dim
        self.hq, self.hkv, self.d = model.hq_local, model.hkv_local, d
        self.qkv_cols = (self.hq + 2 * self.hkv) * d
        H, I = c.hidden, c.ffn // model.tp_size
        R = max_rows
        e = lambda *s: torch.empty(*s, dtype=BF, device=dev)
        self.x, self.xn, self.delta = e(R, H), e(R, H), e(R, H)
        self.qkv, self.attn = e(R, self.qkv_cols), e(R, self.hq * d)
        self.gu, self.act = e(R, 2 * I), e(R, I)
        self.vocab_local = c.vocab // model.tp_size
        self.max_logit_rows = min(R, 256)
        self.logits = torch.empty(self.max_logit_rows, self.vocab_local, dtype=torch.float32, device=dev)
        self.pick_id = torch.zeros(self.max_logit_rows, dtype=torch.int32, device=dev)
        self.pick_val = torch.zeros(self.max_logit_rows, dtype=torch.float32, device=dev)
        self.scale = 1.0 / math.sqrt(d)
        self.decode_splits = decode_splits
        self.att_ml = torch.empty(R * self.hq * decode_splits * 2, dtype=torch.float32, device=dev)
        self.att_acc = torch.empty(min(R, 256) * self.hq * decode_splits * d, dtype=torch.float32, device=dev)
        self.ws = ops.default_workspace(dev)

    # ------------------------------------------------------------------
    def forward(self, rows: int, tokens, positions, row_req, logits_rows: Optional[slice] = None,
                decode: bool = False, pick: bool = True):
        """Run `rows` rows through the model.  tokens/positions/row_req: int32 device tensors [rows].
        Logits (fp32, this rank's vocab slice) are produced for `logits_rows` (default: all rows when
        decode, else only the last row) and the greedy pick of those rows lands in self.pick_id."""
        m, c, kv = self.m, self.m.cfg, self.kv
        x, xn, delta = self.x[:rows], self.xn[:rows], self.delta[:rows]
        qkv, attn, gu, act = self.qkv[:rows], self.attn[:rows], self.gu[:rows], self.act[:rows]
        ops.embed_gather(tokens, m.embed, out=x)
        have_delta = False
        splits = self.decode_splits if (decode and rows <= 256) else 1
        for li, L in enumerate(m.layers):
            ops.rmsnorm(x, L.in_norm, c.eps, delta=delta if have_delta else None, out=xn)
            ops.linear(xn, L.qkv, out=qkv)
            cache = kv.layers[li]
            ops.rope_kv_write(qkv, positions, row_req, kv.block_table, m.inv_freq, cache, self.hq, self.hkv, self.d,
                              rot_dim=c.rot_dim or self.d, mscale=m.mscale, q_norm_w=L.q_norm, k_norm_w=L.k_norm,
                              eps=c.eps)
            self.attention(qkv, cache, row_req, positions, rows, splits, attn)
            ops.linear(attn, L.o, out=delta)
            if self.reducer is not None:
                self.reducer.all_reduce(delta)
            ops.rmsnorm(x, L.post_norm, c.eps, delta=delta, out=xn)
            ops.linear(xn, L.gate_up, out=gu)
            ops.swiglu(gu, out=act)
            ops.linear(act, L.down, out=delta)
            if self.reducer is not None:
                self.reducer.all_reduce(delta)
            have_delta = True
        ops.rmsnorm(x, m.final_norm, c.eps, delta=delta if have_delta else None, out=xn)
        if logits_rows is None:
            logits_rows = slice(0, rows) if decode else slice(rows - 1, rows)
        hx = xn[logits_rows]
        n = hx.shape[0]
        assert n <= self.max_logit_rows
        logits = self.logits[:n]
        ops.gemm_tc(hx, m.head, out32=logits)
        if pick:
            ops.argmax(logits, id_base=m.tp_rank * self.vocab_local, out_id=self.pick_id[:n],
                       out_val=self.pick_val[:n])
            if self.reducer is not None and m.tp_size > 1:
                self.reducer.merge_picks(self.pick_id[:n], self.pick_val[:n])
        return logits

    def attention(self, qkv, cache, row_req, positions, rows, splits, out):
        """Attention of `rows` query rows against the paged cache (their own K/V already appended)."""
        if splits > 1:
            ops.attn_decode(qkv, qkv.stride(0), cache, self.kv.block_table, row_req, positions, self.hq, self.hkv,
                            self.d, self.scale, splits=splits, scratch=(self.att_ml, self.att_acc), out=out)
        else:
            ops.attn_decode(qkv, qkv.stride(0), cache, self.kv.block_table, row_req, positions, self.hq, self.hkv,
                            self.d, self.scale, splits=1, out=out)
