"""Prefill / decode plumbing shared by the smaller family runners: chunked prefill of one request, batched decode with
one CUDA graph per batch width (static id / position / request tensors; recurrent state saved around warm-up and
capture so that only replays move the model), paged KV reservation, full-attention rows on the tensor-core kernels.
A subclass provides `forward(tokens, positions, row_req, chunk_slot, all_logits, pos0)` and, if it keeps state besides
the KV cache, `_state_tensors()` and `_reset_state(slot)`.
(reference counterparts: src/engine/graph_engine.hpp capture / replay, src/engine/paged_blocks.hpp.)
"""
from __future__ import annotations

import math
from typing import List, Optional

import torch

from ..ops import core as ops


class RowRunner:
    def _init_rows(self, slots: int, device, kv_layers: int = 0, kv_heads: int = 0, q_heads: int = 0, head_dim: int = 0,
                   page: int = 64, max_seq_len: int = 0, max_rows: int = 0) -> None:
        from ..engine.kv_cache import PagedKV

        self.dev, self.slots, self.max_rows = device, slots, max_rows
        self.lengths = [0] * slots
        self.use_graphs, self._graphs, self._static = True, {}, {}
        self.pdl_graphs = True      # programmatic-dependent-launch edges between this library's kernels in captured passes
        self.kv = None
        if kv_layers:
            blocks_per = (max_seq_len + page - 1) // page + 1
            self.kv = PagedKV(kv_layers, kv_heads, head_dim, slots * blocks_per + 2, slots, blocks_per, page, True, device)
            self.att_q, self.att_kv, self.att_d = q_heads, kv_heads, head_dim
            self.att_scale = 1.0 / math.sqrt(head_dim)
            self.tc_attn = (torch.device(device).type == "cuda" and head_dim in (128, 256)
                            and q_heads // kv_heads in (1, 2, 4, 8))
            if self.tc_attn:
                r, sp = min(max_rows, 32), 32
                self.att_scratch = (torch.empty(r * q_heads * sp * 2, dtype=torch.float32, device=device),
                                    torch.empty(r * q_heads * sp * head_dim, dtype=torch.float32, device=device))

    # ---- hooks
    def _state_tensors(self):
        return []

    def _reset_state(self, slot: int) -> None:
        pass

    def forward(self, tokens, positions, row_req, chunk_slot=None, all_logits=True, pos0=None, extra=None):
        raise NotImplementedError

    def _extra_rows(self, slots: List[int], tokens: List[int], prefill_slot: Optional[int] = None) -> List[List[int]]:
        """Further int32 rows a pass needs per token (they ride in the same static tensor as ids / positions / requests and
        reach `forward` as `extra`).  prefill_slot given: `tokens` are consecutive tokens of that request."""
        return []

    def _note_tokens(self, slot: int, tokens: List[int]) -> None:
        """Called after `tokens` were appended to request `slot`."""

    # ---- full attention over the paged FP8 cache
    def _attention_rows(self, cache_layer: int, qkv: torch.Tensor, positions, row_req, inv_freq, chunk_slot, pos0,
                        out: torch.Tensor) -> torch.Tensor:
        """qkv [rows, (hq + 2 hkv) d] bf16: rotary embedding, K/V append (FP8), causal attention of every row up to its
        own position -> out [rows, hq d].  Prefill chunks and up to 32 decode rows run on the tcgen05 kernels."""
        hq, hkv, d = self.att_q, self.att_kv, self.att_d
        rows = qkv.shape[0]
        cache = self.kv.layers[cache_layer]
        ops.rope_kv_write(qkv, positions, row_req, self.kv.block_table, inv_freq, cache, hq, hkv, d)
        if self.tc_attn and chunk_slot is not None and pos0 is not None:
            ops.attn_prefill_tc(qkv, qkv.stride(0), cache, self.kv.block_table[chunk_slot], pos0, hq, hkv, d,
                                self.att_scale, out=out, rows=rows)
        elif self.tc_attn and rows <= 32:
            splits = max(1, min(32, -(-160 // (hkv * rows))))
            ops.attn_decode_tc(qkv, qkv.stride(0), cache, self.kv.block_table, row_req, positions, hq, hkv, d,
                               self.att_scale, splits=splits, scratch=self.att_scratch, out=out)
        else:
            ops.attn_decode(qkv, qkv.stride(0), cache, self.kv.block_table, row_req, positions, hq, hkv, d,
                            self.att_scale, out=out)
        return out

    # ---- requests
    def reset(self, slot: int) -> None:
        if self.kv is not None:
            self.kv.release(slot)
        self.lengths[slot] = 0
        self._reset_state(slot)

    @torch.no_grad()
    def prefill(self, slot: int, tokens: List[int], chunk: int = 64) -> torch.Tensor:
        """Appends `tokens` to request `slot`; returns the logits of the last token [1, V]."""
        start = self.lengths[slot]
        if self.kv is not None:
            assert self.kv.reserve(slot, start + len(tokens)), "KV pool exhausted"
        out = None
        for o in range(0, len(tokens), chunk):
            part = tokens[o:o + chunk]
            t = torch.tensor(part, dtype=torch.int32, device=self.dev)
            pos = torch.arange(start + o, start + o + len(part), dtype=torch.int32, device=self.dev)
            req = torch.full((len(part),), slot, dtype=torch.int32, device=self.dev)
            ex = self._extra_rows([slot], part, prefill_slot=slot)
            ex = torch.tensor(ex, dtype=torch.int32, device=self.dev) if ex else None
            out = self.forward(t, pos, req, chunk_slot=slot, all_logits=False, pos0=start + o, extra=ex)
            self._note_tokens(slot, part)
        self.lengths[slot] = start + len(tokens)
        return out

    @torch.no_grad()
    def decode(self, slots: List[int], tokens: List[int]) -> torch.Tensor:
        """One token for every listed request -> fp32 logits [len(slots), V]."""
        b = len(slots)
        positions = [self.lengths[s] for s in slots]
        if self.kv is not None:
            for s in slots:
                assert self.kv.reserve(s, self.lengths[s] + 1), "KV pool exhausted"
        host = torch.tensor([tokens, positions, slots] + self._extra_rows(slots, tokens), dtype=torch.int32)
        rest = lambda t: t[3:] if t.shape[0] > 3 else None
        if not (self.use_graphs and torch.device(self.dev).type == "cuda"):
            d = host.to(self.dev)
            out = self.forward(d[0], d[1], d[2], extra=rest(d))
        else:
            st = self._static.get(b)
            if st is None:
                st = self._static[b] = torch.zeros(host.shape[0], b, dtype=torch.int32, device=self.dev)
            st.copy_(host, non_blocking=True)
            g = self._graphs.get(b)
            if g is None:
                saved = [t.clone() for t in self._state_tensors()]
                side = torch.cuda.Stream()
                side.wait_stream(torch.cuda.current_stream())
                with torch.cuda.stream(side):
                    self.forward(st[0], st[1], st[2], extra=rest(st))
                torch.cuda.current_stream().wait_stream(side)
                torch.cuda.synchronize()
                from ..engine.graph import capture_with_pdl
                graph, out, _ = capture_with_pdl(lambda: self.forward(st[0], st[1], st[2], extra=rest(st)), self.pdl_graphs)
                for t, s0 in zip(self._state_tensors(), saved):
                    t.copy_(s0)
                g = self._graphs[b] = (graph, out)
            graph, out = g
            graph.replay()
        for s, t in zip(slots, tokens):
            self.lengths[s] += 1
            self._note_tokens(s, [t])
        return out
