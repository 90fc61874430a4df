"""Offline generation engine: chunked prefill + CUDA-graph decode loop over the paged KV pool.

Public use::

    model  = DenseModel.random_init(DenseConfig.dense_27b(), device="cuda")
    engine = LLMEngine(model, max_batch=8, max_seq_len=34816)
    out    = engine.generate(prompts, max_tokens=256)        # list[list[int]]

Decode runs as one captured graph per batch width.  A replay needs no host input: the graph ends
with a bookkeeping kernel that feeds the picked ids back as the next tokens, advances positions and
appends the ids to a device ring, so N steps are N graph launches with a single readback (or one
pinned readback per step when tokens are streamed).
(reference behaviour: src/engine/graph_engine.hpp:1827-2995 step_batch / launch / settle_front.)
"""
from __future__ import annotations

import time
from typing import List, Optional, Sequence

import torch

from ..models.dense import DenseModel
from ..ops import _lib
from ..ops._lib import call, ptr, stream_ptr
from .graph import NativeGraph
from .kv_cache import PagedKV
from .runner import DenseRunner


class LLMEngine:
    def __init__(self, model: DenseModel, max_batch: int = 8, max_seq_len: int = 4096, prefill_chunk: int = 2048,
                 kv_blocks: Optional[int] = None, reducer=None, use_graphs: bool = True, ring_steps: int = 1024,
                 decode_pdl: bool = True, act_terms: int = 3, fuse_ar: bool = True, fused_decode: Optional[bool] = None,
                 options=None):
        c = model.cfg
        self.model, self.max_batch, self.max_seq_len = model, max_batch, max_seq_len
        self.prefill_chunk = prefill_chunk
        self.dev = model.embed.device
        page = c.page
        max_blocks_per_req = (max_seq_len + page - 1) // page
        if kv_blocks is None:
            kv_blocks = max_blocks_per_req * max_batch
        self.kv = PagedKV(c.layers, model.hkv_local, c.head_dim, kv_blocks, max_batch, max_blocks_per_req, page,
                          c.kv_fp8, self.dev)
        rows = max(prefill_chunk, max_batch)
        # split-KV decode attention: one wave of CTAs (two resident per SM) is the sweet spot -- measured at 8 rows x 8 kv
        # heads: 13.6 us with 4 splits at ctx 2048 (17.6 us with 8), 33 us with 4 at ctx 8192 (49 us with 16)
        splits = max(1, min(16, 296 // max(1, model.hkv_local * max_batch)))
        from .options import EngineOptions
        self.options = options or EngineOptions()
        self.options.apply_process_wide()
        if self.options.decode_splits > 0:
            splits = self.options.decode_splits
        if fused_decode is None:
            fused_decode = self.options.layer_kernel
        self.decode_pdl = decode_pdl
        self.runner = DenseRunner(model, self.kv, rows, reducer=reducer, decode_splits=splits, decode_rows=max_batch,
                                  act_terms=act_terms, fuse_ar=fuse_ar, fused_decode=fused_decode,
                                  l2_prefetch=self.options.l2_prefetch, fuse_combine=self.options.fuse_combine,
                                  seq_parallel=self.options.seq_parallel)
        self.use_graphs = use_graphs
        self.ring_steps = ring_steps
        i32 = dict(dtype=torch.int32, device=self.dev)
        self.d_tokens = torch.zeros(max_batch, **i32)
        self.d_positions = torch.zeros(max_batch, **i32)
        self.d_row_req = torch.arange(max_batch, **i32)
        self.d_ring = torch.zeros(ring_steps * max_batch, **i32)
        self.d_step = torch.zeros(1, **i32)
        self.p_tokens = torch.zeros(rows, **i32)
        self.p_positions = torch.zeros(rows, **i32)
        self.p_row_req = torch.zeros(rows, **i32)
        self.h_tokens = torch.zeros(rows, dtype=torch.int32).pin_memory() if self.dev.type == "cuda" else None
        self.h_ring = torch.zeros(ring_steps * max_batch, dtype=torch.int32).pin_memory() \
            if self.dev.type == "cuda" else None
        self.h_step_out = torch.zeros(max_batch, dtype=torch.int32).pin_memory() if self.dev.type == "cuda" else None
        self.h_step_in = torch.zeros(max_batch, dtype=torch.int32).pin_memory() if self.dev.type == "cuda" else None
        self.graphs = {}
        self._h2d_done = None
        self.lengths = [0] * max_batch
        self.kernel_launches = 0

    # ------------------------------------------------------------------ prefill
    @torch.no_grad()
    def prefill(self, slot: int, tokens: Sequence[int] | torch.Tensor, start_pos: int = 0,
                embed_spans=None) -> torch.Tensor:
        """Prefill request `slot` with `tokens` (host ints) at positions start_pos.. ; returns the device
        tensor holding the greedy first token (int32, shape [1]).  embed_spans: [(absolute start position, bf16 rows
        [n, hidden] on the device)] whose rows replace the token embeddings of the positions they cover (images)."""
        n = len(tokens)
        self.runner.embed_spans = embed_spans
        assert start_pos + n <= self.max_seq_len
        if not self.kv.reserve(slot, start_pos + n):
            raise RuntimeError("KV pool exhausted")
        host = torch.as_tensor(tokens, dtype=torch.int32)
        done = 0
        r = self.runner
        while done < n:
            t = min(self.prefill_chunk, n - done)
            if self.h_tokens is not None:
                # the pinned staging buffer is reused by every chunk: wait until the previous chunk's copy has left it
                if self._h2d_done is not None:
                    self._h2d_done.synchronize()
                self.h_tokens[:t].copy_(host[done:done + t])
                self.p_tokens[:t].copy_(self.h_tokens[:t], non_blocking=True)
                if self._h2d_done is None:
                    self._h2d_done = torch.cuda.Event()
                self._h2d_done.record()
            else:
                self.p_tokens[:t].copy_(host[done:done + t])
            torch.arange(start_pos + done, start_pos + done + t, dtype=torch.int32, device=self.dev,
                         out=self.p_positions[:t])
            self.p_row_req[:t].fill_(slot)
            r.forward(t, self.p_tokens[:t], self.p_positions[:t], self.p_row_req[:t], decode=False,
                      chunk=(slot, start_pos + done))
            done += t
        self.lengths[slot] = start_pos + n
        r.embed_spans = None
        return r.pick_id[:1]

    @torch.no_grad()
    def prefill_group(self, pieces) -> torch.Tensor:
        """Runs of prompt tokens of SEVERAL requests in one pass: pieces = [(slot, tokens, start_pos, last), ...] with at
        most `prefill_chunk` tokens in total.  Every row attends through the per-row attention kernel (its request, its
        position), so the pass reads the weights once for all requests.  Returns the greedy first tokens of the pieces
        marked `last`, in piece order (int32 device tensor)."""
        total = sum(len(t) for _, t, _, _ in pieces)
        assert 1 <= total <= self.prefill_chunk
        toks, pos, req, lasts = [], [], [], []
        for slot, t, start, last in pieces:
            n = len(t)
            assert start + n <= self.max_seq_len
            if not self.kv.reserve(slot, start + n):
                raise RuntimeError("KV pool exhausted")
            toks += list(t)
            pos += list(range(start, start + n))
            req += [slot] * n
            if last:
                lasts.append(len(toks) - 1)
            self.lengths[slot] = start + n
        host = torch.tensor([toks, pos, req], dtype=torch.int32)
        self.p_tokens[:total].copy_(host[0])
        self.p_positions[:total].copy_(host[1])
        self.p_row_req[:total].copy_(host[2])
        r = self.runner
        r.embed_spans = None
        idx = torch.tensor(lasts or [total - 1], dtype=torch.long, device=self.dev)
        r.forward(total, self.p_tokens[:total], self.p_positions[:total], self.p_row_req[:total], decode=False, chunk=None,
                  logits_rows=idx)
        return r.pick_id[:len(lasts)]

    # ------------------------------------------------------------------ decode
    def _decode_body(self, b: int):
        r = self.runner
        r.forward(b, self.d_tokens[:b], self.d_positions[:b], self.d_row_req[:b], decode=True)
        call("dgpp_decode_advance", ptr(r.pick_id), ptr(self.d_tokens), ptr(self.d_positions), ptr(self.d_ring),
             ptr(self.d_step), b, self.ring_steps, stream_ptr())

    def _graph(self, b: int):
        g = self.graphs.get(b)
        if g is None:
            # warm up outside capture (lazy func attributes, tensor-map encoder lookup), then restore state
            saved = (self.d_tokens.clone(), self.d_positions.clone(), self.d_step.clone(), self.d_ring.clone())
            s = torch.cuda.Stream()
            s.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(s):
                self._decode_body(b)
            torch.cuda.current_stream().wait_stream(s)
            torch.cuda.synchronize()
            self.d_tokens.copy_(saved[0]); self.d_positions.copy_(saved[1])
            self.d_step.copy_(saved[2]); self.d_ring.copy_(saved[3])
            g = NativeGraph(lambda: self._decode_body(b), pdl=self.decode_pdl)
            self.graphs[b] = g
        return g

    def set_adapter(self, adapter) -> None:
        """Install (or with None remove) a bound low-rank adapter.  Captured decode graphs are dropped: the
        adapted and the plain step are different launch sequences."""
        self.runner.lora = adapter
        self.graphs.clear()

    def launches_per_step(self, b: Optional[int] = None) -> int:
        """Kernel launches of this package inside one decode step: the kernel-node count of the captured graph of
        batch width `b` (any captured width when b is None); without a captured graph, the launch sequence counted
        from the runner's layer walk."""
        if self.graphs:
            g = self.graphs.get(b) if b is not None else None
            g = g or next(iter(self.graphs.values()))
            return int(g.kernel_nodes)
        c = self.model.cfg
        r = self.runner
        if r.decode_fp4:
            per_layer = 10 + (1 if r.decode_splits > 1 else 0)          # 4 quantisers, 4 GEMMs, rope / append, attention
            if r.reducer is not None and not r.fuse_ar:
                per_layer += 2 * r.reducer.launches_per_all_reduce
        else:
            per_layer = 9 + (1 if r.decode_splits > 1 else 0)
            if r.reducer is not None:
                per_layer += 2 * r.reducer.launches_per_all_reduce
        return 1 + c.layers * per_layer + 4

    @torch.no_grad()
    def start_decode(self, slots: Sequence[int], first_tokens: torch.Tensor) -> None:
        """Arm the decode state: request slot i decodes in batch row i (slots must be 0..b-1)."""
        b = len(slots)
        assert list(slots) == list(range(b)), "decode rows are the first b request slots"
        self.d_tokens[:b].copy_(first_tokens[:b])
        pos = torch.tensor([self.lengths[s] for s in slots], dtype=torch.int32)
        self.d_positions[:b].copy_(pos)
        self.d_step.zero_()

    @torch.no_grad()
    def decode_step(self, b: int) -> None:
        """One decode step for batch rows 0..b-1 (asynchronous)."""
        if self.use_graphs and self.dev.type == "cuda":
            self._graph(b).replay()
        else:
            self._decode_body(b)

    @torch.no_grad()
    def generate(self, prompts: List[List[int]], max_tokens: int = 32, stream_tokens: bool = False,
                 timings: Optional[dict] = None, native_loop: bool = False, stop_ids=(), inflight: int = 2) -> List[List[int]]:
        """Greedy generation for up to max_batch prompts.  With `stream_tokens` every step's ids are read
        back through pinned memory before the next step is launched (what a streaming server does).
        native_loop: the step loop runs in the native executor (no per-token Python): up to `inflight` graph replays
        outstanding, ids and device status read back per step, rows watched for `stop_ids` (a row's output ends with
        its stop id; the loop ends when every row has stopped)."""
        b = len(prompts)
        assert 1 <= b <= self.max_batch
        for s in range(b):
            self.kv.release(s)
        firsts = torch.zeros(b, dtype=torch.int32, device=self.dev)
        t0 = time.perf_counter()
        for s, p in enumerate(prompts):
            if not self.kv.reserve(s, len(p) + max_tokens + 1):
                raise RuntimeError("KV pool exhausted")
            firsts[s:s + 1].copy_(self.prefill(s, p))
        if timings is not None:
            torch.cuda.synchronize() if self.dev.type == "cuda" else None
            timings["prefill_s"] = time.perf_counter() - t0
        out = [[int(x)] for x in firsts.tolist()]
        self.start_decode(list(range(b)), firsts)
        steps = max_tokens - 1
        t1 = time.perf_counter()
        if native_loop and self.use_graphs and self.dev.type == "cuda" and steps > 0:
            ids, row_stop, launched = self._graph(b).decode_loop(self.d_tokens, b, steps, inflight, tuple(stop_ids))
            ids = ids.tolist()
            for s in range(b):
                last = row_stop[s] if row_stop[s] >= 0 else len(ids) - 1
                out[s] += [ids[i][s] for i in range(last + 1)]
            steps = launched            # the device bookkeeping advanced once per launched step
        elif stream_tokens and self.h_step_out is not None:
            # host-owned token stream: each step's input ids go host -> device from pinned memory (the host
            # may have rewritten them, e.g. grammar or stop handling), the picked ids come back the same way
            for s in range(b):
                self.h_step_in[s] = out[s][-1]
            for i in range(steps):
                self.d_tokens[:b].copy_(self.h_step_in[:b], non_blocking=True)
                self.decode_step(b)
                self.h_step_out[:b].copy_(self.d_tokens[:b], non_blocking=True)
                torch.cuda.current_stream().synchronize()
                for s in range(b):
                    t = int(self.h_step_out[s])
                    out[s].append(t)
                    self.h_step_in[s] = t
        else:
            done = 0
            while done < steps:
                n = min(self.ring_steps, steps - done)
                self.d_step.zero_()
                for _ in range(n):
                    self.decode_step(b)
                ring = self.d_ring[:n * b].view(n, b).cpu() if self.h_ring is None else None
                if ring is None:
                    self.h_ring[:n * self.max_batch].copy_(self.d_ring[:n * self.max_batch], non_blocking=True)
                    torch.cuda.current_stream().synchronize()
                    ring = self.h_ring[:n * b].view(n, b)
                for i in range(n):
                    for s in range(b):
                        out[s].append(int(ring[i, s]))
                done += n
        if timings is not None:
            timings["decode_s"] = time.perf_counter() - t1
            timings["decode_steps"] = steps
        for s in range(b):
            self.lengths[s] += steps
        return out
