"""Cold tier for KV blocks: an engine wrapper that spills full, hash-identified KV blocks to the NVMe disk tier when
their last reference goes away and restores them at the start of a later prefill instead of recomputing them.

The wrapper sits between the scheduler and a block-paged engine.  It needs three things from the wrapped engine:
``read_block(block) -> bytes`` / ``write_block(block, bytes)`` (all layers' K/V, scales included, of one block) and
``advance(slot, tokens)`` (declare that many positions of the slot filled without running them).  Identity of a block
is the prefix cache's own chain hash (FNV-1a over the parent hash and the block's token ids), which the wrapper
recomputes from the tokens it sees: prompt chunks arrive through ``prefill``, generated tokens through ``step_batch``,
and attached prefix blocks carry the hash recorded when they were filled.

* spill: ``release_block`` / ``close`` of a block whose reference count is about to reach zero and whose hash is
  known -> ``DiskTier.put_async(hash, bytes)``.
* restore: ``prefill`` at a block-aligned position walks the chunk's full blocks; while the tier holds the block's
  hash the bytes are written into the slot's (already reserved) block and the tokens are skipped.  At least one token
  is always left to run, because the scheduler wants the logits of the last prompt position.
A restored block is byte-identical to the one that was computed (CRC-checked pages), so generation is unchanged.

Keys on disk are the chain hash mixed with a 64-bit FINGERPRINT of what computed the block (`cache_fingerprint`: model
configuration, a digest of the weights, KV format and layout, tensor-parallel rank and size, adapter).  A tier
directory adopted by a server with other weights, another quantisation or another shard therefore holds nothing
under this engine's keys, instead of handing back KV that another model computed.
(reference counterparts: src/engine/nvme_tier.hpp spill / restore of KV pages, src/sched/scheduler.cpp disk pump,
 src/sched/disk_cache.cpp.)
"""
from __future__ import annotations

import hashlib
import json
from typing import Dict, List, Optional

from ..runtime import rt

_M64 = (1 << 64) - 1


def cache_fingerprint(**identity) -> int:
    """64-bit digest of everything that determines the bytes of a KV block besides its tokens.  Pass whatever
    applies, e.g. ``cache_fingerprint(config=dataclasses.asdict(cfg), weights=weights_digest(model), kv="fp8-e4m3/64",
    tp=(rank, size), adapter=adapter_sha)``; values must be JSON-serialisable (tuples become lists)."""
    blob = json.dumps(identity, sort_keys=True, default=str).encode()
    return int.from_bytes(hashlib.blake2b(blob, digest_size=8).digest(), "little")


def weights_digest(tensors, sample_bytes: int = 1 << 16) -> str:
    """Cheap identity of a set of weight tensors: shapes, dtypes and the first / last `sample_bytes` of each."""
    import torch

    h = hashlib.blake2b(digest_size=16)
    for t in tensors:
        if t is None:
            continue
        h.update(repr((tuple(t.shape), str(t.dtype))).encode())
        flat = t.detach().reshape(-1).view(torch.uint8)
        n = min(sample_bytes, flat.numel())
        h.update(flat[:n].cpu().numpy().tobytes())
        h.update(flat[flat.numel() - n:].cpu().numpy().tobytes())
    return h.hexdigest()


class SpillingEngine(rt.SchedulerEngine):
    def __init__(self, base, tier, fingerprint: Optional[int] = None):
        super().__init__()
        self.b, self.tier = base, tier
        if fingerprint is None:
            f = getattr(base, "cache_fingerprint", None)
            fingerprint = f() if f else 0
        self.fp = int(fingerprint) & _M64
        self.bt = base.block_tokens()
        n = base.max_concurrent()
        self.block_hash: Dict[int, int] = {}          # physical block -> chain hash of the prefix ending with it
        self.slot_hash: List[int] = [rt.FNV_SEED] * n  # chain hash at the slot's last block boundary
        self.slot_tail: List[List[int]] = [[] for _ in range(n)]   # tokens after that boundary
        self.slot_len = [0] * n
        self.spilled = self.restored = self.restored_tokens = 0
        self._last: Dict[int, int] = {}

    # ---- pass-through geometry
    def max_concurrent(self): return self.b.max_concurrent()
    def block_tokens(self): return self.bt
    def total_blocks(self): return self.b.total_blocks()
    def free_blocks(self): return self.b.free_blocks()
    def max_context(self): return self.b.max_context()
    def max_tokens_per_step(self):
        f = getattr(self.b, "max_tokens_per_step", None)
        return f() if f else 1
    def reserve(self, slot, tokens): return self.b.reserve(slot, tokens)
    def slot_blocks(self, slot): return self.b.slot_blocks(slot)
    def retain_block(self, b): self.b.retain_block(b)
    def block_refcount(self, b): return self.b.block_refcount(b)
    def usable_prefix(self, blocks):
        f = getattr(self.b, "usable_prefix", None)
        return f(list(blocks)) if f else len(blocks)

    def open(self, slot, request_id):
        f = getattr(self.b, "open", None)
        if f:
            f(slot, request_id)

    def key(self, h: int) -> int:
        """Disk key of the block whose chain hash is h: the hash mixed with this engine's fingerprint."""
        x = (h ^ self.fp) & _M64
        x = (x * 0x9E3779B97F4A7C15 + (self.fp >> 7)) & _M64
        return x ^ (x >> 29)

    # ---- hashing of what a slot holds
    def _note(self, slot: int, tokens: List[int]) -> None:
        """Account tokens that now have KV in the slot; record the hash of every block they complete."""
        tail = self.slot_tail[slot]
        tail.extend(tokens)
        blocks = None
        while len(tail) >= self.bt:
            h = rt.chain_hash(self.slot_hash[slot], tail[:self.bt])
            del tail[:self.bt]
            if blocks is None:
                blocks = self.b.slot_blocks(slot)
            idx = self.slot_len[slot] // self.bt
            if idx < len(blocks):
                self.block_hash[blocks[idx]] = h
            self.slot_hash[slot] = h
            self.slot_len[slot] += self.bt

    def attach_prefix(self, slot, blocks):
        blocks = list(blocks)
        self.b.attach_prefix(slot, blocks)
        h = self.block_hash.get(blocks[-1])
        self.slot_len[slot] = len(blocks) * self.bt
        self.slot_tail[slot] = []
        # an attached block without a recorded hash (published before this wrapper saw it) stops restores for the
        # slot: without the parent hash the following blocks cannot be identified
        self.slot_hash[slot] = h if h is not None else None

    # ---- spill
    def _maybe_spill(self, block: int) -> None:
        h = self.block_hash.get(block)
        if h is None or self.b.block_refcount(block) != 1:
            return
        if not self.tier.contains(self.key(h)):
            self.tier.put_async(self.key(h), self.b.read_block(block))
            self.spilled += 1
        del self.block_hash[block]

    def release_block(self, b):
        self._maybe_spill(b)
        self.b.release_block(b)

    def close(self, slot):
        for blk in self.b.slot_blocks(slot):
            self._maybe_spill(blk)
        self.b.close(slot)
        self.slot_hash[slot] = rt.FNV_SEED
        self.slot_tail[slot] = []
        self.slot_len[slot] = 0

    # ---- execution
    def prefill(self, slot, tokens, pos, last):
        tokens = list(tokens)
        if pos == 0:
            self.slot_hash[slot], self.slot_tail[slot], self.slot_len[slot] = rt.FNV_SEED, [], 0
        skip = 0
        if self.slot_hash[slot] is not None and not self.slot_tail[slot] and pos % self.bt == 0 and pos == self.slot_len[slot]:
            blocks = self.b.slot_blocks(slot)
            h = self.slot_hash[slot]
            while len(tokens) - skip > self.bt or (not last and len(tokens) - skip == self.bt):
                ids = tokens[skip:skip + self.bt]
                hb = rt.chain_hash(h, ids)
                idx = (pos + skip) // self.bt
                if idx >= len(blocks) or not self.tier.contains(self.key(hb)):
                    break
                data = self.tier.get(self.key(hb))
                if data is None:                      # failed its checks on the way back: compute instead
                    break
                self.b.write_block(blocks[idx], data)
                self.block_hash[blocks[idx]] = hb
                h = hb
                skip += self.bt
            if skip:
                self.b.advance(slot, skip)
                self.slot_hash[slot] = h
                self.slot_len[slot] += skip
                self.restored += skip // self.bt
                self.restored_tokens += skip
        if skip == len(tokens):
            return -1                                 # (only when not `last`: every token of the chunk was restored)
        tok = self.b.prefill(slot, tokens[skip:], pos + skip, last)
        if self.slot_hash[slot] is not None:
            self._note(slot, tokens[skip:])
        if last:
            self._last[slot] = tok
        return tok

    def step_batch(self, slots):
        slots = list(slots)
        out = self.b.step_batch(slots)
        for s, toks in zip(slots, out):
            if self.slot_hash[s] is not None:
                # the token fed into this pass (the previous pending one) and all but the last new token have KV now
                fed = [self._last[s]] + list(toks[:-1])
                self._note(s, fed)
            self._last[s] = toks[-1]
        return out
