"""Bump arenas over a few large slabs: every long-lived buffer of an engine (activations, scratch, KV pages, pinned
staging) is a view into a slab of its memory class, so nothing allocates on the hot path and the engine's footprint
is one number per class.

Classes: ``device_hot`` (touched every step: activations, scratch), ``device_cold`` (KV pages, snapshots),
``host_pinned`` (staging for H2D / D2H copies).  Allocation is a 256-byte aligned bump; there is no free -- an arena
is released as a whole (`reset`).  A request that does not fit opens another slab of at least `slab_bytes`.
``named_streams`` is the matching pool of CUDA streams by name.
(reference counterparts: src/core/arena.hpp MemClass DeviceHot / DeviceCold / HostPinned slab allocator,
 src/core/streams.hpp named stream pool.)
"""
from __future__ import annotations

from typing import Dict, List, Sequence

import torch

ALIGN = 256
CLASSES = ("device_hot", "device_cold", "host_pinned")


class Arena:
    def __init__(self, device="cuda", slab_bytes: int = 256 << 20):
        self.device = torch.device(device)
        self.slab_bytes = slab_bytes
        self._slabs: Dict[str, List[torch.Tensor]] = {c: [] for c in CLASSES}
        self._used: Dict[str, int] = {c: 0 for c in CLASSES}     # bytes used in the newest slab
        self.allocations: Dict[str, int] = {c: 0 for c in CLASSES}

    def _new_slab(self, mem_class: str, nbytes: int) -> torch.Tensor:
        n = max(self.slab_bytes, nbytes)
        if mem_class == "host_pinned":
            pin = self.device.type == "cuda" and torch.cuda.is_available()
            slab = torch.empty(n, dtype=torch.uint8, pin_memory=pin)
        else:
            slab = torch.empty(n, dtype=torch.uint8, device=self.device)
        self._slabs[mem_class].append(slab)
        self._used[mem_class] = 0
        return slab

    def alloc(self, shape: Sequence[int], dtype: torch.dtype, mem_class: str = "device_hot", zero: bool = False) -> torch.Tensor:
        if mem_class not in self._slabs:
            raise KeyError(f"unknown memory class {mem_class!r}")
        numel = 1
        for s in shape:
            numel *= int(s)
        nbytes = numel * torch.empty(0, dtype=dtype).element_size()
        slabs = self._slabs[mem_class]
        if not slabs or self._used[mem_class] + nbytes > slabs[-1].numel():
            self._new_slab(mem_class, nbytes)
        slab = self._slabs[mem_class][-1]
        o = self._used[mem_class]
        self._used[mem_class] = (o + nbytes + ALIGN - 1) // ALIGN * ALIGN
        self.allocations[mem_class] += 1
        t = slab[o:o + nbytes].view(dtype).view(*shape)
        if zero:
            t.zero_()
        return t

    def reserved_bytes(self, mem_class: str) -> int:
        return sum(s.numel() for s in self._slabs[mem_class])

    def used_bytes(self, mem_class: str) -> int:
        slabs = self._slabs[mem_class]
        return sum(s.numel() for s in slabs[:-1]) + (self._used[mem_class] if slabs else 0)

    def report(self) -> Dict[str, Dict[str, int]]:
        return {c: {"slabs": len(self._slabs[c]), "reserved": self.reserved_bytes(c), "used": self.used_bytes(c),
                    "allocations": self.allocations[c]} for c in CLASSES}

    def reset(self) -> None:
        for c in CLASSES:
            self._slabs[c].clear()
            self._used[c] = 0
            self.allocations[c] = 0


class named_streams:
    """Streams by name, created on first use (`named_streams(device)["copy"]`)."""

    def __init__(self, device="cuda"):
        self.device = torch.device(device)
        self._s: Dict[str, "torch.cuda.Stream"] = {}

    def __getitem__(self, name: str):
        if name not in self._s:
            self._s[name] = torch.cuda.Stream(device=self.device)
        return self._s[name]

    def names(self) -> List[str]:
        return sorted(self._s)
