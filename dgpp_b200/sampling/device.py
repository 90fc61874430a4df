"""Device sampler front end: packs per-row sampling parameters, owns the count table / scratch, launches
``csrc/kernels/sample.cu`` and finishes rows the device could not resolve with the host oracle (wider prefixes).
(reference counterparts: src/kernels/sample_pick.cu launch wrappers, src/engine/tp_bus.hpp sampling folds.)"""
from __future__ import annotations

import ctypes as C
import struct
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence

import torch

from ..ops import _lib
from ..ops._lib import I, L, P, call, ptr, stream_ptr

_lib.declare("dgpp_sample", [P, L, P, P, P, P, P, P, P, P, P, P, P, P, P, I, I, I, P])
_lib.declare("dgpp_sample_local", [P, L, P, P, P, P, P, P, P, P, P, P, I, I, I, I, I, P])
_lib.declare("dgpp_sample_merge", [P, P, P, P, P, P, P, P, P, P, I, I, I, P])
_lib.declare("dgpp_sample_count_tokens", [P, I, I, P, I, I, P])
_lib.declare("dgpp_sample_count_step", [P, I, P, P, I, P])

ROW_FMT = "<6f4i2Q"          # SampleRow in sample.cu
ROW_BYTES = struct.calcsize(ROW_FMT)
MAX_TOP, MAX_BIAS, MAX_CAND = 20, 512, 256


@dataclass
class SamplingParams:
    temperature: float = 0.0
    top_k: int = 0
    top_p: float = 1.0
    min_p: float = 0.0
    repetition_penalty: float = 1.0
    presence_penalty: float = 0.0
    frequency_penalty: float = 0.0
    seed: int = 0
    top_logprobs: int = 0
    logit_bias: Dict[int, float] = field(default_factory=dict)

    @property
    def greedy(self) -> bool:
        return self.temperature <= 0.0 or self.top_p <= 0.0


@dataclass
class Sampled:
    token: int
    logprob: float
    top: List[tuple]
    on_device: bool


class DeviceSampler:
    def __init__(self, vocab: int, max_rows: int, slots: int, device, candidates: int = 128):
        assert 1 <= candidates <= MAX_CAND
        lib = _lib.load()
        assert lib.dgpp_sample_row_bytes() == ROW_BYTES, "SampleRow layout drifted from ROW_FMT"
        self.vocab, self.max_rows, self.slots, self.dev, self.candidates = vocab, max_rows, slots, device, candidates
        f32 = dict(dtype=torch.float32, device=device)
        i32 = dict(dtype=torch.int32, device=device)
        self.counts = torch.zeros(slots, vocab, **i32)
        self.z = torch.empty(max_rows, vocab, **f32)
        self.parts = torch.empty(max_rows, (vocab + 255) // 256, 2, **f32)
        self.rows_dev = torch.zeros(max_rows, ROW_BYTES, dtype=torch.uint8, device=device)
        self.rows_host = torch.zeros(max_rows, ROW_BYTES, dtype=torch.uint8).pin_memory() if device.type == "cuda" else None
        self.bias_ids = torch.full((max_rows, MAX_BIAS), -1, **i32)
        self.bias_vals = torch.zeros(max_rows, MAX_BIAS, **f32)
        self.out_token = torch.zeros(max_rows, **i32)
        self.out_logprob = torch.zeros(max_rows, **f32)
        self.out_flags = torch.zeros(max_rows, **i32)
        self.out_top_ids = torch.zeros(max_rows, MAX_TOP, **i32)
        self.out_top_lp = torch.zeros(max_rows, MAX_TOP, **f32)
        self.out_top_n = torch.zeros(max_rows, **i32)
        self._host_counts: List[Dict[int, int]] = [dict() for _ in range(slots)]

    # ---- token counts (penalties)
    def reset_slot(self, slot: int) -> None:
        self.counts[slot].zero_()
        self._host_counts[slot] = {}

    def count(self, slot: int, ids: Sequence[int], delta: int = 1) -> None:
        if not len(ids):
            return
        t = torch.as_tensor(list(ids), dtype=torch.int32).to(self.dev)
        call("dgpp_sample_count_tokens", ptr(self.counts), self.vocab, slot, ptr(t), t.numel(), delta, stream_ptr())
        hc = self._host_counts[slot]
        for i in ids:
            hc[int(i)] = hc.get(int(i), 0) + delta

    # ---- one sampling pass
    def sample(self, logits: torch.Tensor, params: Sequence[SamplingParams], slots: Sequence[int],
               positions: Sequence[int], masks: Optional[torch.Tensor] = None, count_picks: bool = True) -> List[Sampled]:
        """logits: fp32 [rows, >= vocab] on the device.  masks: optional uint32 [rows, ceil(vocab/32)] allowed bits."""
        rows = len(params)
        assert rows <= self.max_rows and logits.dtype == torch.float32 and logits.shape[0] >= rows
        any_bias = any(p.logit_bias for p in params)
        packed = bytearray()
        for r, (p, slot, pos) in enumerate(zip(params, slots, positions)):
            nb = min(len(p.logit_bias), MAX_BIAS)
            packed += struct.pack(ROW_FMT, p.temperature, p.top_p, p.min_p, p.repetition_penalty, p.presence_penalty,
                                  p.frequency_penalty, p.top_k, p.top_logprobs, slot, nb, p.seed & (2 ** 64 - 1), pos)
            if nb:
                items = sorted(p.logit_bias.items())[:nb]
                self.bias_ids[r, :nb] = torch.tensor([k for k, _ in items], dtype=torch.int32)
                self.bias_vals[r, :nb] = torch.tensor([v for _, v in items], dtype=torch.float32)
        blob = torch.frombuffer(packed, dtype=torch.uint8).view(rows, ROW_BYTES)
        if self.rows_host is not None:
            self.rows_host[:rows].copy_(blob)
            self.rows_dev[:rows].copy_(self.rows_host[:rows], non_blocking=True)
        else:
            self.rows_dev[:rows].copy_(blob)
        call("dgpp_sample", ptr(logits), logits.stride(0), ptr(self.rows_dev), ptr(self.counts),
             ptr(self.bias_ids) if any_bias else None, ptr(self.bias_vals) if any_bias else None, ptr(masks),
             ptr(self.z), ptr(self.parts), ptr(self.out_token), ptr(self.out_logprob), ptr(self.out_flags),
             ptr(self.out_top_ids), ptr(self.out_top_lp), ptr(self.out_top_n), rows, self.vocab, self.candidates,
             stream_ptr())
        tok = self.out_token[:rows].tolist()
        lp = self.out_logprob[:rows].tolist()
        flags = self.out_flags[:rows].tolist()
        need_top = any(p.top_logprobs for p in params)
        tn = self.out_top_n[:rows].tolist() if need_top else [0] * rows
        tids = self.out_top_ids[:rows].tolist() if need_top else None
        tlps = self.out_top_lp[:rows].tolist() if need_top else None
        out: List[Sampled] = []
        for r in range(rows):
            if flags[r]:
                top = [(tids[r][i], tlps[r][i]) for i in range(tn[r])] if need_top else []
                out.append(Sampled(tok[r], lp[r], top, True))
            else:
                out.append(self._host_finish(logits[r, :self.vocab], params[r], slots[r], positions[r],
                                             None if masks is None else masks[r]))
        if count_picks:
            for r, s in enumerate(out):
                if slots[r] >= 0:
                    self.count(slots[r], [s.token])
        return out

    # ---- vocabulary-sharded head (tensor parallel): candidate tables instead of a logits gather
    def _pack_rows(self, params, slots, positions) -> bool:
        rows = len(params)
        any_bias = any(p.logit_bias for p in params)
        packed = bytearray()
        for r, (p, slot, pos) in enumerate(zip(params, slots, positions)):
            nb = min(len(p.logit_bias), MAX_BIAS)
            packed += struct.pack(ROW_FMT, p.temperature, p.top_p, p.min_p, p.repetition_penalty, p.presence_penalty,
                                  p.frequency_penalty, p.top_k, p.top_logprobs, slot, nb, p.seed & (2 ** 64 - 1), pos)
            if nb:
                items = sorted(p.logit_bias.items())[:nb]
                self.bias_ids[r, :nb] = torch.tensor([k for k, _ in items], dtype=torch.int32)
                self.bias_vals[r, :nb] = torch.tensor([v for _, v in items], dtype=torch.float32)
        blob = torch.frombuffer(packed, dtype=torch.uint8).view(rows, ROW_BYTES)
        if self.rows_host is not None:
            self.rows_host[:rows].copy_(blob)
            self.rows_dev[:rows].copy_(self.rows_host[:rows], non_blocking=True)
        else:
            self.rows_dev[:rows].copy_(blob)
        return any_bias

    def local_tables(self, logits_slice: torch.Tensor, id_base: int, params, slots, positions, masks=None):
        """Step 1 on this rank's slice [id_base, id_base + width) of the vocabulary: returns (cand [rows, C] int64 keys,
        ms [rows, 2] fp32, nt [rows] int32).  `self.vocab` is the FULL vocabulary (count table, bias ids, mask bits)."""
        rows, width = len(params), logits_slice.shape[1]
        any_bias = self._pack_rows(params, slots, positions)
        cand = torch.zeros(rows, self.candidates, dtype=torch.int64, device=self.dev)
        ms = torch.zeros(rows, 2, dtype=torch.float32, device=self.dev)
        nt = torch.zeros(rows, dtype=torch.int32, device=self.dev)
        call("dgpp_sample_local", ptr(logits_slice), logits_slice.stride(0), ptr(self.rows_dev), ptr(self.counts),
             ptr(self.bias_ids) if any_bias else None, ptr(self.bias_vals) if any_bias else None, ptr(masks), ptr(self.z),
             ptr(self.parts), ptr(cand), ptr(ms), ptr(nt), rows, width, id_base, self.vocab, self.candidates, stream_ptr())
        return cand, ms, nt

    def merge_tables(self, cands, mss, nts, params, slots, count_picks: bool = True) -> List[Sampled]:
        """Step 2: the ranks' tables stacked in rank order ([world, rows, ...]); every rank computes the same picks.
        A row whose draw does not resolve inside the candidate prefix comes back with resolved=False (the caller
        gathers that row's logits and finishes it on the host)."""
        world, rows = cands.shape[0], cands.shape[1]
        call("dgpp_sample_merge", ptr(self.rows_dev), ptr(cands.contiguous()), ptr(mss.contiguous()), ptr(nts.contiguous()),
             ptr(self.out_token), ptr(self.out_logprob), ptr(self.out_flags), ptr(self.out_top_ids), ptr(self.out_top_lp),
             ptr(self.out_top_n), rows, world, self.candidates, stream_ptr())
        tok, lp, flags = self.out_token[:rows].tolist(), self.out_logprob[:rows].tolist(), self.out_flags[:rows].tolist()
        need_top = any(p.top_logprobs for p in params)
        tn = self.out_top_n[:rows].tolist() if need_top else [0] * rows
        tids = self.out_top_ids[:rows].tolist() if need_top else None
        tlps = self.out_top_lp[:rows].tolist() if need_top else None
        out = []
        for r in range(rows):
            top = [(tids[r][i], tlps[r][i]) for i in range(tn[r])] if (need_top and flags[r]) else []
            out.append(Sampled(tok[r], lp[r], top, bool(flags[r])))
        if count_picks:
            for r, sm in enumerate(out):
                if slots[r] >= 0 and sm.on_device:
                    self.count(slots[r], [sm.token])
        return out

    def sample_sharded(self, logits_slice: torch.Tensor, id_base: int, params, slots, positions, group=None, masks=None,
                       count_picks: bool = True) -> List[Sampled]:
        """Sampling on a vocabulary-sharded head without gathering the logits: per-rank candidate tables (a few KB per
        row) are all-gathered and folded identically on every rank.  Rows that do not resolve inside the candidate
        prefix gather their logits and finish on the host (rare: top_p close to 1 on a flat distribution)."""
        import torch.distributed as dist

        world = dist.get_world_size(group)
        cand, ms, nt = self.local_tables(logits_slice, id_base, params, slots, positions, masks)
        gc = torch.empty(world, *cand.shape, dtype=cand.dtype, device=self.dev)
        gm = torch.empty(world, *ms.shape, dtype=ms.dtype, device=self.dev)
        gn = torch.empty(world, *nt.shape, dtype=nt.dtype, device=self.dev)
        dist.all_gather_into_tensor(gc, cand, group=group)
        dist.all_gather_into_tensor(gm, ms, group=group)
        dist.all_gather_into_tensor(gn, nt, group=group)
        out = self.merge_tables(gc, gm, gn, params, slots, count_picks=False)
        for r, sm in enumerate(out):
            if not sm.on_device:
                part = logits_slice[r:r + 1].contiguous()
                parts = [torch.empty_like(part) for _ in range(world)]
                dist.all_gather(parts, part, group=group)
                full = torch.cat(parts, dim=1)[0]
                out[r] = self._host_finish(full[:self.vocab], params[r], slots[r], positions[r], None if masks is None else masks[r])
        if count_picks:
            for r, sm in enumerate(out):
                if slots[r] >= 0:
                    self.count(slots[r], [sm.token])
        return out

    def _host_finish(self, logits_row, p: SamplingParams, slot: int, pos: int, mask_row) -> Sampled:
        from ..runtime import rt

        allowed = None
        if mask_row is not None:
            bits = mask_row.cpu().numpy().view("uint32")
            allowed = [int((bits[i >> 5] >> (i & 31)) & 1) for i in range(self.vocab)]
        counts = self._host_counts[slot] if slot >= 0 else {}
        tok, lp, top = rt.sample_reference(logits_row.cpu().tolist(), p.temperature, p.top_k, p.top_p, p.min_p,
                                           p.repetition_penalty, p.presence_penalty, p.frequency_penalty, p.seed,
                                           p.top_logprobs, p.logit_bias, counts, pos, allowed, self.candidates)
        return Sampled(tok, lp, list(top), False)
