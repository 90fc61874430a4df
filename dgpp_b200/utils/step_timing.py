"""Per-step device timing slots: ``DGPP_STEP_TIMING=1`` (or ``StepTimer(enabled=True)``) brackets named phases of
an engine step with CUDA events on the launching stream and accumulates their device time.

Slots follow the phases the engine distinguishes: step (whole pass), prefill, decode, attn, moe, fold (collective),
pick (LM head + sampling), sync (final host wait).  Events are recorded, never synchronised, inside the step;
`collect()` resolves finished pairs after the step's own synchronisation, so timing adds no host wait of its own.
Off by default: an idle timer costs one attribute test per phase.  Without a GPU the timer falls back to the host
clock so the plumbing is testable.
(reference counterpart: src/engine/step_timing.hpp cudaEvent slots kStep / kMoe / kMoeSync / kFoldDrain / kFold /
 kPick / kFinalSync, surfaced as the `timings` extension of API responses.)
"""
from __future__ import annotations

import contextlib
import os
import time
from typing import Dict, List, Tuple

import torch

SLOTS = ("step", "prefill", "decode", "attn", "moe", "fold", "pick", "sync")


class StepTimer:
    def __init__(self, enabled: bool | None = None, use_cuda: bool | None = None):
        if enabled is None:
            enabled = os.environ.get("DGPP_STEP_TIMING", "") not in ("", "0")
        self.enabled = enabled
        self.cuda = torch.cuda.is_available() if use_cuda is None else use_cuda
        self.total_ms: Dict[str, float] = {s: 0.0 for s in SLOTS}
        self.count: Dict[str, int] = {s: 0 for s in SLOTS}
        self._open: List[Tuple[str, object, object]] = []
        self._pool: List[object] = []

    def _event(self):
        return self._pool.pop() if self._pool else torch.cuda.Event(enable_timing=True)

    @contextlib.contextmanager
    def phase(self, slot: str):
        if not self.enabled:
            yield
            return
        if slot not in self.total_ms:
            raise KeyError(f"unknown timing slot {slot!r}")
        if self.cuda:
            a, b = self._event(), self._event()
            a.record()
            try:
                yield
            finally:
                b.record()
                self._open.append((slot, a, b))
        else:
            t0 = time.perf_counter()
            try:
                yield
            finally:
                self.total_ms[slot] += (time.perf_counter() - t0) * 1e3
                self.count[slot] += 1

    def collect(self) -> None:
        """Fold the event pairs that have completed into the totals (call after the step's synchronisation)."""
        if not self.cuda:
            return
        keep = []
        for slot, a, b in self._open:
            if b.query():
                self.total_ms[slot] += a.elapsed_time(b)
                self.count[slot] += 1
                self._pool += [a, b]
            else:
                keep.append((slot, a, b))
        self._open = keep

    def timings(self, reset: bool = False) -> Dict[str, Dict[str, float]]:
        """{slot: {"ms": total, "n": count, "mean_ms": ...}} for the slots that were hit."""
        self.collect()
        out = {s: {"ms": round(self.total_ms[s], 4), "n": self.count[s],
                   "mean_ms": round(self.total_ms[s] / self.count[s], 4)} for s in SLOTS if self.count[s]}
        if reset:
            for s in SLOTS:
                self.total_ms[s], self.count[s] = 0.0, 0
        return out
