"""Paged KV pool: device planes per layer plus the shared block table.

One int32 table ``[max_requests, max_blocks_per_request]`` is shared by all layers and planes
(K, V, their FP8 scales); a block holds ``page`` tokens.  Block bookkeeping (free list, refcounts
for prefix sharing) is done by the native ``PagedBlockTable`` of the runtime when it is built,
with an equivalent pure-Python fallback.
(reference: src/engine/paged_blocks.hpp:1-215 -- one table shared by all cache planes, LIFO free list.)
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional

import torch


@dataclass
class KVLayer:
    k: torch.Tensor
    v: torch.Tensor
    k_scale: Optional[torch.Tensor]
    v_scale: Optional[torch.Tensor]
    page: int
    fp8: bool


class _PyBlockTable:
    """LIFO free list + refcounts (fallback when the native runtime is not built)."""

    def __init__(self, num_blocks: int):
        self.free = list(range(num_blocks - 1, -1, -1))
        self.ref = [0] * num_blocks

    def alloc(self) -> int:
        if not self.free:
            return -1
        b = self.free.pop()
        self.ref[b] = 1
        return b

    def retain(self, b: int) -> None:
        self.ref[b] += 1

    def release(self, b: int) -> None:
        self.ref[b] -= 1
        if self.ref[b] == 0:
            self.free.append(b)

    def free_count(self) -> int:
        return len(self.free)


class PagedKV:
    def __init__(self, layers: int, hkv: int, d: int, num_blocks: int, max_requests: int, max_blocks_per_req: int,
                 page: int = 64, fp8: bool = True, device="cuda"):
        self.layers_n, self.hkv, self.d, self.page, self.fp8 = layers, hkv, d, page, fp8
        self.num_blocks, self.max_requests, self.max_blocks = num_blocks, max_requests, max_blocks_per_req
        dt = torch.uint8 if fp8 else torch.bfloat16
        self.layers: List[KVLayer] = []
        for _ in range(layers):
            k = torch.zeros(num_blocks, hkv, page, d, dtype=dt, device=device)
            v = torch.zeros(num_blocks, hkv, page, d, dtype=dt, device=device)
            ks = torch.ones(num_blocks, hkv, page, dtype=torch.float32, device=device) if fp8 else None
            vs = torch.ones(num_blocks, hkv, page, dtype=torch.float32, device=device) if fp8 else None
            self.layers.append(KVLayer(k, v, ks, vs, page, fp8))
        self.block_table = torch.zeros(max_requests, max_blocks_per_req, dtype=torch.int32, device=device)
        self.host_table = torch.zeros(max_requests, max_blocks_per_req, dtype=torch.int32)
        self.req_blocks: List[List[int]] = [[] for _ in range(max_requests)]
        try:
            from ..runtime import rt
            self.alloc = rt.PagedBlockTable(num_blocks)
        except Exception:  # native runtime not built
            self.alloc = _PyBlockTable(num_blocks)

    @staticmethod
    def bytes_per_block(layers: int, hkv: int, d: int, page: int, fp8: bool) -> int:
        per = hkv * page * d * (1 if fp8 else 2) + (hkv * page * 4 if fp8 else 0)
        return 2 * layers * per

    def reserve(self, req: int, tokens: int) -> bool:
        """Make sure request slot `req` owns blocks covering `tokens` positions."""
        need = (tokens + self.page - 1) // self.page
        have = len(self.req_blocks[req])
        if need > self.max_blocks:
            return False
        if need - have > self.alloc.free_count():
            return False
        changed = False
        while have < need:
            b = self.alloc.alloc()
            self.req_blocks[req].append(b)
            self.host_table[req, have] = b
            have += 1
            changed = True
        if changed:
            self.block_table[req].copy_(self.host_table[req], non_blocking=True)
        return True

    def attach(self, req: int, blocks: List[int]) -> None:
        """Share already-filled blocks (prefix hit): refcount them and list them first."""
        assert not self.req_blocks[req]
        for i, b in enumerate(blocks):
            self.alloc.retain(b)
            self.req_blocks[req].append(b)
            self.host_table[req, i] = b
        self.block_table[req].copy_(self.host_table[req], non_blocking=True)

    def release(self, req: int) -> None:
        for b in self.req_blocks[req]:
            self.alloc.release(b)
        self.req_blocks[req] = []

    def free_blocks(self) -> int:
        return self.alloc.free_count()
