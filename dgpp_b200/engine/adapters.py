"""Scheduler-facing engines: implementations of the native ``SchedulerEngine`` contract.

* ``ReferenceEngine`` -- runs ``DenseModel.forward_reference`` (pure PyTorch, any device, optional gloo / NCCL
  tensor parallelism) over a block-paged KV store, so the scheduler, the prefix cache (block sharing by
  reference count) and multi-rank agreement can be exercised without a GPU.
* ``KernelEngine``    -- the sm_100a path: ``LLMEngine`` prefill chunks and CUDA-graph decode steps.

Both keep KV in blocks of ``block_tokens`` positions handed out by the native ``PagedBlockTable``; attaching a
cached prefix only bumps reference counts.
(contract: csrc/rt/scheduler.h ``SchedulerEngine``; reference counterpart src/engine/eager_engine.hpp:49-999,
 src/engine/graph_engine.hpp:233.)
"""
from __future__ import annotations

import time
from typing import List, Optional

import torch

from ..models.dense import DenseModel
from ..runtime import rt


class EmbedSplice:
    """Per-request input-embedding overrides (image rows), shared by the engines behind the scheduler.

    The serving layer computes an image's rows with the vision tower and registers them under the request id before it
    submits the request; the scheduler's `open(slot, id)` binds them to the slot, and every prefill chunk of the slot
    hands the spans to the model, which writes them over the token embeddings of the covered positions.  Towards the
    scheduler an image position carries a pseudo token id >= vocab derived from the image's content hash, so that the
    prefix cache tells two images apart; `_real_ids` maps those ids to the family's image pad id before they reach
    the embedding table.  (reference counterparts: src/models/*/image_prefill.cpp, the image embedding splice in
    run_rows, src/serve/vision_frontend.cpp span bookkeeping.)"""

    def _splice_init(self, slots: int, vocab: int, pad_id: int = 0) -> None:
        self._embeds_by_id = {}
        self._slot_embeds = [None] * slots
        self._vocab, self._pad_id = vocab, pad_id

    def set_embeds(self, request_id: str, spans) -> None:
        """spans: [(start position in the prompt, rows [n, hidden])]."""
        self._embeds_by_id[request_id] = list(spans)

    def _splice_open(self, slot: int, request_id: str) -> None:
        # kept until forget(): a request shed back to the queue is opened again under the same id
        self._slot_embeds[slot] = self._embeds_by_id.get(request_id)

    def _splice_forget(self, request_id: str) -> None:
        self._embeds_by_id.pop(request_id, None)

    def forget(self, request_id: str) -> None:
        """Drops the per-request registrations of a retired request."""
        self._splice_forget(request_id)

    def _real_ids(self, tokens):
        v, pad = self._vocab, self._pad_id
        return [t if t < v else pad for t in tokens]


class EngineFailure(RuntimeError):
    """The device reported a failed bounded wait (or another unrecoverable condition): the engine's buffers are not
    trustworthy any more.  The serving loop answers every open request with an engine_failure error and stops."""


class ReferenceEngine(EmbedSplice, rt.SchedulerEngine):
    def __init__(self, model: DenseModel, slots: int = 4, num_blocks: int = 256, block_tokens: int = 16,
                 max_context: int = 1024, all_reduce=None):
        super().__init__()
        self.m, self.slots_n, self.bt, self.maxctx = model, slots, block_tokens, max_context
        self.table = rt.PagedBlockTable(num_blocks)
        c = model.cfg
        dev = model.embed.device
        shape = (c.layers, num_blocks, block_tokens, model.hkv_local, c.head_dim)
        self.k = torch.zeros(shape, dtype=torch.float32, device=dev)
        self.v = torch.zeros(shape, dtype=torch.float32, device=dev)
        self.blocks: List[List[int]] = [[] for _ in range(slots)]
        self.filled = [0] * slots
        self.pending: List[Optional[int]] = [None] * slots
        self.all_reduce = all_reduce
        self._splice_init(slots, c.vocab)

    def open(self, slot, request_id):
        self._splice_open(slot, request_id)

    # ---- geometry
    def max_concurrent(self):
        return self.slots_n

    def block_tokens(self):
        return self.bt

    def total_blocks(self):
        return self.table.num_blocks()

    def free_blocks(self):
        return self.table.free_count()

    def max_context(self):
        return self.maxctx

    # ---- blocks
    def reserve(self, slot, tokens):
        need = (tokens + self.bt - 1) // self.bt
        if need - len(self.blocks[slot]) > self.table.free_count():
            return False
        while len(self.blocks[slot]) < need:
            self.blocks[slot].append(self.table.alloc())
        return True

    def attach_prefix(self, slot, blocks):
        assert not self.blocks[slot]
        for b in blocks:
            self.table.retain(b)
            self.blocks[slot].append(b)
        self.filled[slot] = len(blocks) * self.bt

    def slot_blocks(self, slot):
        return list(self.blocks[slot])

    def retain_block(self, b):
        self.table.retain(b)

    def release_block(self, b):
        self.table.release(b)

    def block_refcount(self, b):
        return self.table.refcount(b)

    def close(self, slot):
        for b in self.blocks[slot]:
            self.table.release(b)
        self.blocks[slot] = []
        self.filled[slot] = 0
        self.pending[slot] = None

    # ---- cold tier hooks (engine.spill.SpillingEngine)
    def read_block(self, b: int) -> bytes:
        return torch.stack([self.k[:, b], self.v[:, b]]).contiguous().cpu().numpy().tobytes()

    def write_block(self, b: int, data: bytes) -> None:
        t = torch.frombuffer(bytearray(data), dtype=torch.float32).view(2, *self.k[:, b].shape).to(self.k.device)
        self.k[:, b], self.v[:, b] = t[0], t[1]

    def advance(self, slot: int, tokens: int) -> None:
        self.filled[slot] += tokens

    # ---- compute
    def _run(self, slot: int, tokens: List[int]) -> int:
        c = self.m.cfg
        n0 = self.filled[slot]
        idx = torch.tensor(self.blocks[slot], dtype=torch.long, device=self.k.device)
        kv = []
        for li in range(c.layers):
            if n0:
                k = self.k[li, idx].reshape(-1, self.m.hkv_local, c.head_dim)[:n0]
                v = self.v[li, idx].reshape(-1, self.m.hkv_local, c.head_dim)[:n0]
                kv.append((k, v))
            else:
                kv.append(None)
        logits, kv = self.m.forward_reference(torch.tensor(self._real_ids(tokens), device=self.k.device), start_pos=n0,
                                              kv=kv, all_reduce=self.all_reduce, embed_spans=self._slot_embeds[slot])
        n1 = n0 + len(tokens)
        pos = torch.arange(n0, n1, device=self.k.device)
        blk = idx[pos // self.bt]
        off = pos % self.bt
        for li in range(c.layers):
            self.k[li, blk, off] = kv[li][0][n0:n1]
            self.v[li, blk, off] = kv[li][1][n0:n1]
        self.filled[slot] = n1
        row = logits[-1].float()
        if self.all_reduce is not None and self.m.tp_size > 1:
            return self._sharded_pick(row)
        return int(torch.argmax(row))  # first maximal index = lowest id

    def _sharded_pick(self, row: torch.Tensor) -> int:
        import torch.distributed as dist

        v, i = torch.max(row, 0)
        vl = self.m.cfg.vocab // self.m.tp_size
        mine = torch.tensor([float(v), float(int(i) + self.m.tp_rank * vl)], dtype=torch.float64)
        allv = [torch.zeros_like(mine) for _ in range(self.m.tp_size)]
        dist.all_gather(allv, mine)
        best = 0
        for r in range(1, self.m.tp_size):
            if allv[r][0] > allv[best][0]:
                best = r
        return int(allv[best][1])

    def prefill(self, slot, tokens, pos, last):
        assert pos == self.filled[slot], (pos, self.filled[slot])
        tok = self._run(slot, list(tokens))
        if last:
            self.pending[slot] = tok
            return tok
        return -1

    def step_batch(self, slots):
        out = []
        for s in slots:
            tok = self._run(s, [self.pending[s]])
            self.pending[s] = tok
            out.append([tok])
        return out


class KernelEngine(EmbedSplice, rt.SchedulerEngine):
    """The CUDA engine behind the scheduler: chunked prefill and graph-replayed decode for arbitrary slot sets."""

    def __init__(self, engine, spec_drafts: int = 0):
        """spec_drafts > 0: greedy speculative decoding with context-lookup drafts.  Every decode pass carries, per
        request, its pending token plus up to `spec_drafts` proposed continuations as extra rows of the same batch;
        the rows' own greedy picks verify the drafts (longest matching prefix + one bonus token), so the output is
        token for token what plain greedy decoding gives.  Rejected positions are simply overwritten later: the
        dense family has no state besides the KV cache.  (reference counterparts: src/engine/speculative.hpp
        GreedySpeculator / judge_verify, src/engine/lookup_draft.hpp, verify rows batched into the decode pass.)"""
        super().__init__()
        self.e = engine
        self.kv = engine.kv
        self.spec_k = max(0, int(spec_drafts))
        self.drafts = [rt.LookupDraft(2, 4) for _ in range(engine.max_batch)] if self.spec_k else None
        self.schedule = [rt.VerifySchedule(0, self.spec_k, min(self.spec_k, 3)) for _ in range(engine.max_batch)] \
            if self.spec_k else None
        self.spec_graphs = {}
        self.spec_proposed = self.spec_accepted = 0
        self.pending = [None] * engine.max_batch
        self._splice_init(engine.max_batch, engine.model.cfg.vocab)
        self.filled = [0] * engine.max_batch
        b = engine.max_batch
        hb = max(b, engine.runner.max_logit_rows if self.spec_k else b)
        self.h_tok = torch.zeros(hb, dtype=torch.int32).pin_memory()
        self.h_pos = torch.zeros(hb, dtype=torch.int32).pin_memory()
        self.h_req = torch.zeros(hb, dtype=torch.int32).pin_memory()
        self.h_out = torch.zeros(hb, dtype=torch.int32).pin_memory()
        if self.spec_k:
            dev = engine.dev
            self.s_tok = torch.zeros(hb, dtype=torch.int32, device=dev)
            self.s_pos = torch.zeros(hb, dtype=torch.int32, device=dev)
            self.s_req = torch.zeros(hb, dtype=torch.int32, device=dev)
        self.poll_status = True                        # read the device status block after every step (see _poll_device)
        self.step_deadline_s = 120.0                   # host-side bound on one prefill chunk / decode pass
        self.by_id = {}
        self.emitted = {}                              # request id -> tokens the sampler picked for it so far
        self.slot_req = [None] * b
        self.slot_cfg = [None] * b
        self.last_logprobs = [None] * b
        self.sampler = None
        from ..utils.step_timing import StepTimer
        self.timer = StepTimer()                 # DGPP_STEP_TIMING=1 turns the event slots on

    def max_concurrent(self):
        return self.e.max_batch

    def max_tokens_per_step(self):
        return 1 + self.spec_k

    def block_tokens(self):
        return self.kv.page

    def total_blocks(self):
        return self.kv.num_blocks

    def free_blocks(self):
        return self.kv.free_blocks()

    def max_context(self):
        return self.e.max_seq_len

    def reserve(self, slot, tokens):
        return self.kv.reserve(slot, tokens)

    def attach_prefix(self, slot, blocks):
        self.kv.attach(slot, list(blocks))
        self.filled[slot] = len(blocks) * self.kv.page

    def slot_blocks(self, slot):
        return list(self.kv.req_blocks[slot])

    def retain_block(self, b):
        self.kv.alloc.retain(b)

    def release_block(self, b):
        self.kv.alloc.release(b)

    def block_refcount(self, b):
        return self.kv.alloc.refcount(b)

    def close(self, slot):
        self.kv.release(slot)
        self.filled[slot] = 0
        self.pending[slot] = None
        self.slot_cfg[slot] = None

    # ------------------------------------------------------------------ cold tier hooks (engine.spill.SpillingEngine)
    def read_block(self, b: int) -> bytes:
        parts = []
        for L in self.kv.layers:
            for t in (L.k, L.v, L.k_scale, L.v_scale):
                if t is not None:
                    parts.append(t[b].contiguous().view(torch.uint8).reshape(-1))
        return torch.cat(parts).cpu().numpy().tobytes()

    def write_block(self, b: int, data: bytes) -> None:
        flat = torch.frombuffer(bytearray(data), dtype=torch.uint8).to(self.e.dev)
        o = 0
        for L in self.kv.layers:
            for t in (L.k, L.v, L.k_scale, L.v_scale):
                if t is not None:
                    n = t[b].numel() * t.element_size()
                    t[b].copy_(flat[o:o + n].view(t.dtype).view(t[b].shape))
                    o += n
        assert o == flat.numel(), "block image does not match this cache geometry"

    def advance(self, slot: int, tokens: int) -> None:
        self.filled[slot] += tokens

    # ------------------------------------------------------------------ sampling / constraints
    def configure(self, request_id: str, params=None, grammar=None, prompt_ids=None) -> None:
        """Registers sampling parameters (``SamplingParams``), a token grammar (``rt.JsonGrammar``) and the prompt ids
        (for the penalties' token counts) of a request before it is submitted to the scheduler."""
        self.by_id[request_id] = (params, grammar, prompt_ids)

    def forget(self, request_id: str) -> None:
        """Drops what configure() / set_embeds() registered for a request.  The owner of the request calls it when
        the request retires (or is rejected / cancelled while still queued); until then the entries stay, because a
        request shed back to the queue is opened again under the same id and must get the same sampling parameters,
        its grammar in the state its generated tokens left it in, and its image rows."""
        self.by_id.pop(request_id, None)
        self.emitted.pop(request_id, None)
        self._splice_forget(request_id)

    def open(self, slot, request_id):
        self._splice_open(slot, request_id)
        cfg = self.by_id.get(request_id)
        self.slot_cfg[slot] = None
        self.slot_req[slot] = request_id
        self.last_logprobs[slot] = None
        if cfg is None or (cfg[0] is None and cfg[1] is None):
            return
        params, grammar, prompt_ids = cfg
        from ..sampling.device import DeviceSampler, SamplingParams
        if self.sampler is None:
            self.sampler = DeviceSampler(self.e.model.cfg.vocab, self.e.max_batch, self.e.max_batch, self.e.dev)
        self.sampler.reset_slot(slot)
        params = params or SamplingParams()
        if params.repetition_penalty != 1.0 or params.presence_penalty or params.frequency_penalty:
            # token counts of the prompt and, for a re-admitted request, of what it had generated before it was shed
            seen = list(prompt_ids or []) + self.emitted.get(request_id, [])
            if seen:
                self.sampler.count(slot, seen)
        # (the grammar object itself has consumed every token picked so far, so it resumes where the request stopped)
        self.slot_cfg[slot] = (params, grammar)

    def _sample_rows(self, logits, slots):
        """Device sampler over the rows of `slots` (rows of plain greedy slots keep the engine's own pick)."""
        import numpy as np
        from ..sampling.device import SamplingParams
        rows = len(slots)
        params, masks = [], None
        for s in slots:
            cfg = self.slot_cfg[s]
            params.append(cfg[0] if cfg else SamplingParams())
        if any(self.slot_cfg[s] and self.slot_cfg[s][1] is not None for s in slots):
            words = (self.e.model.cfg.vocab + 31) // 32
            m = np.full((rows, words), 0xFFFFFFFF, dtype=np.uint32)
            for r, s in enumerate(slots):
                cfg = self.slot_cfg[s]
                if cfg and cfg[1] is not None:
                    gm = cfg[1].mask()
                    m[r, :] = 0
                    m[r, :min(words, gm.shape[0])] = gm[:words]
            masks = torch.from_numpy(m.view(np.int32)).to(self.e.dev)
        if self.e.model.tp_size > 1:
            # vocabulary-sharded head: every rank builds the candidate table of its slice (a few KB per row), the tables
            # are all-gathered and folded identically on every rank: no logits gather, the same token everywhere
            vl = self.e.runner.vocab_local
            base = self.e.model.tp_rank * vl
            width = max(0, min(vl, self.e.model.cfg.vocab - base))
            picked = self.sampler.sample_sharded(logits[:rows, :width], base, params,
                                                 [s if self.slot_cfg[s] else -1 for s in slots],
                                                 [self.filled[s] for s in slots], masks=masks)
        else:
            picked = self.sampler.sample(logits, params, [s if self.slot_cfg[s] else -1 for s in slots],
                                         [self.filled[s] for s in slots], masks=masks)
        for r, s in enumerate(slots):
            cfg = self.slot_cfg[s]
            if cfg:
                self.last_logprobs[s] = (picked[r].logprob, picked[r].top)
                if cfg[1] is not None:
                    cfg[1].accept(picked[r].token)
                self.emitted.setdefault(self.slot_req[s], []).append(picked[r].token)
        return [p.token for p in picked]

    def _poll_device(self) -> None:
        """Every bounded device wait (pipeline barriers, accumulators, peer flags, grid barriers) reports its expiry
        into the per-device status block instead of trapping.  The serving path reads the block after every prefill
        chunk and decode pass: a non-zero code means that what the kernels left behind cannot be trusted (a peer that
        stopped answering, a lost copy), so the step raises and the owner of the loop fails the engine instead of
        streaming tokens picked from stale buffers.
        (reference behaviour: engine_failure events and exit 2 / 3, src/serve/generation_service.cpp:4300-4486.)"""
        if not self.poll_status or self.e.dev.type != "cuda":
            return
        import ctypes as C
        from ..ops import _lib
        from ..ops import core as _ops
        # the status read below synchronises the device: bound that wait first, so a device that stopped making progress
        # becomes an engine failure instead of a hung serving thread
        if not _ops.stream_wait(self.step_deadline_s):
            raise EngineFailure(f"the device did not finish a step within {self.step_deadline_s:.0f} s")
        buf = (C.c_int * 4)()
        _lib.call("dgpp_status_read", C.cast(buf, C.c_void_p))
        if buf[0] != 0:
            raise EngineFailure(f"device status code={buf[0]} count={buf[1]} detail={buf[2]} "
                                f"(a bounded device wait gave up; see common.h StatusCode)")

    def prefill(self, slot, tokens, pos, last):
        with self.timer.phase("prefill"):
            first = self.e.prefill(slot, self._real_ids(tokens), start_pos=pos, embed_spans=self._slot_embeds[slot])
        self._poll_device()
        self.filled[slot] = pos + len(tokens)
        if self.spec_k:
            if pos == 0:
                self.drafts[slot].reset()
            self.drafts[slot].append(list(tokens))
        if last:
            if self.slot_cfg[slot]:
                tok = self._sample_rows(self.e.runner.logits[:1], [slot])[0]
            else:
                tok = int(first.item())
            self.pending[slot] = tok
            if self.spec_k:
                self.drafts[slot].push(tok)
            return tok
        return -1

    def prefill_group(self, pieces):
        """Several readers in one pass (see LLMEngine.prefill_group).  Requests with sampling settings, speculative
        drafts or embedding spans take the one-request path."""
        pieces = [(s, list(t), p, bool(l)) for s, t, p, l in pieces]
        plain = all(not self.slot_cfg[s] and self._slot_embeds[s] is None for s, _, _, _ in pieces) and not self.spec_k
        if not plain or len(pieces) == 1 or sum(len(t) for _, t, _, _ in pieces) > self.e.prefill_chunk:
            return [self.prefill(s, t, p, l) for s, t, p, l in pieces]
        with self.timer.phase("prefill"):
            firsts = self.e.prefill_group([(s, self._real_ids(t), p, l) for s, t, p, l in pieces])
        self._poll_device()
        firsts = firsts.tolist()
        out, k = [], 0
        for s, t, p, l in pieces:
            self.filled[s] = p + len(t)
            if l:
                tok = int(firsts[k]); k += 1
                self.pending[s] = tok
                out.append(tok)
            else:
                out.append(-1)
        return out

    def mixed_step(self, piece, slots):
        """One pass for a prefill piece and one decode step of `slots`: the piece's rows and one row per decoder (its
        pending token at its next position) go through `LLMEngine.prefill_group` together, so the weights are read once
        and the decoders do not wait behind the chunk.  None (the scheduler then runs the two calls) when a request of
        the pass samples, follows a grammar, carries embedding spans or drafts, or the rows do not fit one pass."""
        s0, toks, pos, last = piece[0], list(piece[1]), piece[2], bool(piece[3])
        slots = list(slots)
        involved = [s0] + slots
        plain = all(not self.slot_cfg[s] and self._slot_embeds[s] is None for s in involved) and not self.spec_k
        if not plain or len(toks) + len(slots) > self.e.prefill_chunk:
            return None
        pieces = [(s0, self._real_ids(toks), pos, last)] + [(s, [self.pending[s]], self.filled[s], True) for s in slots]
        with self.timer.phase("prefill"):
            picks = self.e.prefill_group(pieces).tolist()
        self._poll_device()
        self.filled[s0] = pos + len(toks)
        k, first = 0, -1
        if last:
            first, k = int(picks[0]), 1
            self.pending[s0] = first
        out = []
        for s in slots:
            tok = int(picks[k]); k += 1
            self.filled[s] += 1
            self.pending[s] = tok
            out.append([tok])
        return first, out

    def _spec_graph(self, rows: int):
        """One captured forward per row count (rows = requests + draft rows of this pass)."""
        g = self.spec_graphs.get(rows)
        if g is None:
            from .graph import NativeGraph
            r = self.e.runner
            body = lambda: r.forward(rows, self.s_tok[:rows], self.s_pos[:rows], self.s_req[:rows], decode=True)
            s = torch.cuda.Stream()
            s.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(s):
                body()                                   # warm up outside capture
            torch.cuda.current_stream().wait_stream(s)
            torch.cuda.synchronize()
            g = NativeGraph(body, pdl=self.e.decode_pdl)
            self.spec_graphs[rows] = g
        return g

    def _step_spec(self, slots):
        """Decode pass with draft rows: returns, per slot, the verified tokens (1 .. 1 + drafts)."""
        e, r = self.e, self.e.runner
        cap = min(r.max_logit_rows, r.fp4_rows if r.decode_fp4 else r.max_rows)
        plan, rows = [], 0
        for i, s in enumerate(slots):
            room = cap - rows - (len(slots) - i)             # every later slot still needs its own row
            k = min(self.schedule[s].draft_len(), self.spec_k, max(room, 0),
                    e.max_seq_len - self.filled[s] - 1, len(self.kv.req_blocks[s]) * self.kv.page - self.filled[s] - 1)
            d = self.drafts[s].propose(k) if k > 0 and not self.slot_cfg[s] else []
            toks = [self.pending[s]] + list(d)
            for j, t in enumerate(toks):
                self.h_tok[rows + j] = t
                self.h_pos[rows + j] = self.filled[s] + j
                self.h_req[rows + j] = s
            plan.append((s, rows, d))
            rows += len(toks)
        self.s_tok[:rows].copy_(self.h_tok[:rows], non_blocking=True)
        self.s_pos[:rows].copy_(self.h_pos[:rows], non_blocking=True)
        self.s_req[:rows].copy_(self.h_req[:rows], non_blocking=True)
        with self.timer.phase("decode"):
            if e.use_graphs and e.dev.type == "cuda":
                self._spec_graph(rows).replay()
            else:
                r.forward(rows, self.s_tok[:rows], self.s_pos[:rows], self.s_req[:rows], decode=True)
        self.h_out[:rows].copy_(r.pick_id[:rows], non_blocking=True)
        torch.cuda.current_stream().synchronize()
        self._poll_device()
        out = []
        for s, row0, d in plan:
            if self.slot_cfg[s]:
                tok = self._sample_rows(r.logits[row0:row0 + 1], [s])[0]
                acc = [tok]
            else:
                acc = []
                for j in range(len(d) + 1):
                    t = int(self.h_out[row0 + j])
                    acc.append(t)
                    if j == len(d) or d[j] != t:
                        break
                self.spec_proposed += len(d)
                self.spec_accepted += len(acc) - 1
                if d:
                    self.schedule[s].observe(len(d), len(acc) - 1)
            # the pending token and the accepted drafts now have KV; the last pick is the new pending token.  The
            # drafter's history always ends with the pending token (what follows it is what a draft predicts).
            for t in acc:
                self.drafts[s].push(t)
            self.filled[s] += len(acc)
            self.pending[s] = acc[-1]
            out.append(acc)
        return out

    def step_batch(self, slots):
        if self.spec_k:
            return self._step_spec(list(slots))
        b = len(slots)
        e = self.e
        for i, s in enumerate(slots):
            self.h_tok[i] = self.pending[s]
            self.h_pos[i] = self.filled[s]
            self.h_req[i] = s
        e.d_tokens[:b].copy_(self.h_tok[:b], non_blocking=True)
        e.d_positions[:b].copy_(self.h_pos[:b], non_blocking=True)
        e.d_row_req[:b].copy_(self.h_req[:b], non_blocking=True)
        with self.timer.phase("decode"):
            e.decode_step(b)
        self.h_out[:b].copy_(e.d_tokens[:b], non_blocking=True)
        t_sync = time.perf_counter() if self.timer.enabled else 0.0
        torch.cuda.current_stream().synchronize()
        self._poll_device()
        if self.timer.enabled:
            self.timer.total_ms["sync"] += (time.perf_counter() - t_sync) * 1e3
            self.timer.count["sync"] += 1
            self.timer.collect()
        for s in slots:
            self.filled[s] += 1
        toks = [int(self.h_out[i]) for i in range(b)]
        if any(self.slot_cfg[s] for s in slots):
            sampled = self._sample_rows(e.runner.logits[:b], slots)
            toks = [sampled[i] if self.slot_cfg[s] else toks[i] for i, s in enumerate(slots)]
        out = []
        for i, s in enumerate(slots):
            self.pending[s] = toks[i]
            out.append([toks[i]])
        return out


class HybridEngine(rt.SchedulerEngine):
    """The hybrid (Gated DeltaNet + gated full attention + MoE) runner behind the scheduler.

    A request's state is its paged KV blocks (attention layers) plus one convolution tail and one delta-rule memory
    per GDN layer.  The prefix cache shares KV blocks by hash; the recurrent state cannot be rebuilt from blocks, so
    the engine snapshots it whenever a prefill crosses a multiple of `snapshot_every` tokens and files the snapshot
    under the physical block that ends there (with the block's generation, so a recycled block never matches).
    `usable_prefix` tells the scheduler how much of a matched chain ends on a live snapshot; `attach_prefix` shares
    the blocks and restores that snapshot.  (reference counterparts: src/engine/prefix_arena.hpp state snapshots at
    cut positions, src/models/kda_snapshot.hpp, src/sched/prefix_cache.cpp.)"""

    def __init__(self, runner, snapshot_every: int = 1024, max_snapshots: int = 64, prefill_chunk: int = 256,
                 mtp_depth: int = 0):
        """mtp_depth > 0: every decode step drafts that many tokens with the model's MTP head and verifies them in the
        same pass as the pending token (greedy: the emitted sequence does not change, only how many tokens a step emits)."""
        super().__init__()
        self.r = runner
        self.mtp_depth = mtp_depth
        if mtp_depth:
            runner.enable_spec(mtp_depth)
        self.kv = runner.kv
        page = self.kv.page
        self.snapshot_every = max(page, snapshot_every // page * page)
        self.max_snapshots = max_snapshots
        self.prefill_chunk = prefill_chunk
        self.snaps = {}                 # block id -> (generation, [per GDN layer (conv, ssm)], stamp)
        self.stamp = 0
        self.pending = [None] * len(runner.lengths)
        self.snapshots_taken = self.snapshots_restored = 0

    # ---- geometry
    def max_concurrent(self):
        return len(self.r.lengths)

    def block_tokens(self):
        return self.kv.page

    def total_blocks(self):
        return self.kv.num_blocks

    def free_blocks(self):
        return self.kv.free_blocks()

    def max_context(self):
        return (self.kv.max_blocks - 1) * self.kv.page

    def reserve(self, slot, tokens):
        return self.kv.reserve(slot, tokens)

    def slot_blocks(self, slot):
        return list(self.kv.req_blocks[slot])

    def retain_block(self, b):
        self.kv.alloc.retain(b)

    def release_block(self, b):
        self.kv.alloc.release(b)

    def block_refcount(self, b):
        return self.kv.alloc.refcount(b)

    # ---- snapshots
    def _live(self, block):
        s = self.snaps.get(block)
        if s is None:
            return None
        if s[0] != self.kv.alloc.generation(block) or self.kv.alloc.refcount(block) <= 0:
            del self.snaps[block]
            return None
        return s

    def _snapshot(self, slot, tokens_done):
        block = self.kv.req_blocks[slot][tokens_done // self.kv.page - 1]
        if len(self.snaps) >= self.max_snapshots:
            for b in list(self.snaps):          # (a copy: _live drops dead entries from the dict as it goes)
                self._live(b)
            if len(self.snaps) >= self.max_snapshots:
                oldest = min(self.snaps, key=lambda b: self.snaps[b][2])
                del self.snaps[oldest]
        self.stamp += 1
        state = [st.snapshot(slot) for st in self.r.gdn_state.values()]
        self.snaps[block] = (self.kv.alloc.generation(block), state, self.stamp)
        self.snapshots_taken += 1

    def usable_prefix(self, blocks):
        for j in range(len(blocks), 0, -1):
            if self._live(blocks[j - 1]) is not None:
                return j
        return 0

    def attach_prefix(self, slot, blocks):
        blocks = list(blocks)
        snap = self._live(blocks[-1])
        assert snap is not None, "attach_prefix without a state snapshot at the cut (usable_prefix decides the cut)"
        self.kv.attach(slot, blocks)
        for st, s in zip(self.r.gdn_state.values(), snap[1]):
            st.restore(slot, s)
        self.stamp += 1
        self.snaps[blocks[-1]] = (snap[0], snap[1], self.stamp)
        self.r.lengths[slot] = len(blocks) * self.kv.page
        self.snapshots_restored += 1

    # ---- execution
    def prefill(self, slot, tokens, pos, last):
        tokens = list(tokens)
        if pos == 0 and self.r.lengths[slot] != 0:
            self.close(slot)
        assert self.r.lengths[slot] == pos, (self.r.lengths[slot], pos)
        logits = None
        o = 0
        while o < len(tokens):
            at = pos + o
            to_cut = self.snapshot_every - at % self.snapshot_every
            n = min(len(tokens) - o, to_cut)
            logits = self.r.prefill(slot, tokens[o:o + n], chunk=self.prefill_chunk)
            o += n
            if (pos + o) % self.snapshot_every == 0:
                self._snapshot(slot, pos + o)
        if last:
            tok = int(torch.argmax(logits[0]).item())
            self.pending[slot] = tok
            return tok
        return -1

    def _poll_device(self) -> None:
        """See KernelEngine._poll_device: a non-zero device status after a step fails the engine."""
        if torch.device(getattr(self.r, "dev", "cpu")).type != "cuda":
            return
        import ctypes as C
        from ..ops import _lib
        buf = (C.c_int * 4)()
        _lib.call("dgpp_status_read", C.cast(buf, C.c_void_p))
        if buf[0] != 0:
            raise EngineFailure(f"device status code={buf[0]} count={buf[1]} detail={buf[2]}")

    def step_batch(self, slots):
        slots = list(slots)
        if self.mtp_depth:
            outs = self.r.spec_step(slots, [self.pending[s] for s in slots])
            self._poll_device()
            for s, o in zip(slots, outs):
                self.pending[s] = int(o[-1])
            return [[int(t) for t in o] for o in outs]
        logits = self.r.decode(slots, [self.pending[s] for s in slots])
        toks = torch.argmax(logits[:len(slots)], dim=-1).tolist()
        self._poll_device()
        out = []
        for s, t in zip(slots, toks):
            self.pending[s] = int(t)
            out.append([int(t)])
        return out

    def close(self, slot):
        self.r.reset(slot)
        self.pending[slot] = None


class RunnerEngine(rt.SchedulerEngine):
    """Any family runner with `prefill(slot, tokens, chunk)`, `decode(slots, tokens)`, `reset(slot)` and `lengths` behind
    the scheduler (greedy decoding).  The runner's state (recurrent memories, caches laid out per slot) is not
    addressable by block, so this engine never resumes from the prefix cache: it hands the scheduler a private block
    table for admission arithmetic only and reports no usable prefix.  (reference counterparts: the per-family
    SessionModel adapters of src/engine/session_model.hpp.)"""

    def __init__(self, runner, max_context: int, block_tokens: int = 64, prefill_chunk: int = 256):
        super().__init__()
        self.r, self.bt, self.maxctx, self.prefill_chunk = runner, block_tokens, max_context, prefill_chunk
        n = len(runner.lengths)
        self.per_slot = (max_context + block_tokens - 1) // block_tokens + 1
        self.table = rt.PagedBlockTable(n * self.per_slot + 1)
        self.blocks: List[List[int]] = [[] for _ in range(n)]
        self.pending: List[Optional[int]] = [None] * n

    # ---- geometry
    def max_concurrent(self):
        return len(self.r.lengths)

    def block_tokens(self):
        return self.bt

    def total_blocks(self):
        return self.table.num_blocks()

    def free_blocks(self):
        return self.table.free_count()

    def max_context(self):
        return self.maxctx

    # ---- blocks (accounting only)
    def reserve(self, slot, tokens):
        need = (tokens + self.bt - 1) // self.bt
        if need > self.per_slot or need - len(self.blocks[slot]) > self.table.free_count():
            return False
        while len(self.blocks[slot]) < need:
            self.blocks[slot].append(self.table.alloc())
        return True

    def slot_blocks(self, slot):
        return list(self.blocks[slot])

    def retain_block(self, b):
        self.table.retain(b)

    def release_block(self, b):
        self.table.release(b)

    def block_refcount(self, b):
        return self.table.refcount(b)

    def usable_prefix(self, blocks):
        return 0

    def attach_prefix(self, slot, blocks):
        raise AssertionError("attach_prefix on an engine that reports no usable prefix")

    # ---- execution
    def prefill(self, slot, tokens, pos, last):
        tokens = list(tokens)
        if pos == 0 and self.r.lengths[slot] != 0:
            self.r.reset(slot)
        assert self.r.lengths[slot] == pos, (self.r.lengths[slot], pos)
        logits = self.r.prefill(slot, tokens, chunk=self.prefill_chunk)
        if last:
            self.pending[slot] = int(torch.argmax(logits[-1]).item())
            return self.pending[slot]
        return -1

    def step_batch(self, slots):
        slots = list(slots)
        logits = self.r.decode(slots, [self.pending[s] for s in slots])
        toks = torch.argmax(logits[:len(slots)], dim=-1).tolist()
        if torch.device(getattr(self.r, "dev", "cpu")).type == "cuda":
            import ctypes as C
            from ..ops import _lib
            buf = (C.c_int * 4)()
            _lib.call("dgpp_status_read", C.cast(buf, C.c_void_p))
            if buf[0] != 0:
                raise EngineFailure(f"device status code={buf[0]} count={buf[1]} detail={buf[2]}")
        out = []
        for s, t in zip(slots, toks):
            self.pending[s] = int(t)
            out.append([int(t)])
        return out

    def close(self, slot):
        for b in self.blocks[slot]:
            self.table.release(b)
        self.blocks[slot] = []
        self.pending[slot] = None
        self.r.reset(slot)
