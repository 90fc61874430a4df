"""Resumable cursor over one request of a row engine: feed a prompt in arbitrary pieces, extend token by token, go back
to an earlier position, fork into another slot.

A session owns one slot of an engine that exposes `prefill(slot, tokens, start_pos) -> first greedy token`, a `lengths`
list and a paged KV cache (`kv.reserve / attach / release / req_blocks / page`): `LLMEngine` and anything shaped like
it.  Positions address the KV cache, so going back is bookkeeping: the cursor moves, the blocks stay reserved and the
rows past the cursor are overwritten by whatever is fed next.  A fork shares the FULL blocks in front of the cursor
with the new slot (reference counted) and feeds it the remainder of the last block again.
(reference counterparts: src/engine/session_model.hpp resumable prefill cursor / rollback, src/engine/prefix_arena.hpp
 block sharing.)
"""
from __future__ import annotations

from typing import List, Optional, Sequence


class Session:
    def __init__(self, engine, slot: int):
        self.e, self.slot = engine, slot
        self.tokens: List[int] = []          # every token that has KV, in position order
        self.pending: Optional[int] = None   # greedy pick after the last fed token (has no KV yet)
        engine.kv.release(slot)
        engine.lengths[slot] = 0

    @property
    def position(self) -> int:
        return len(self.tokens)

    def feed(self, tokens: Sequence[int]) -> int:
        """Appends `tokens` at the cursor (any count, the engine chunks them) -> the greedy pick after the last one."""
        tokens = [int(t) for t in tokens]
        if not tokens:
            raise ValueError("feed needs at least one token")
        # rows are written in place: a block that another slot (or the prefix cache) also holds must not change
        page, mine = self.e.kv.page, self.e.kv.req_blocks[self.slot]
        for bi in range(self.position // page, min(len(mine), (self.position + len(tokens) - 1) // page + 1)):
            if self.e.kv.alloc.refcount(mine[bi]) > 1:
                raise RuntimeError(f"position {bi * page}..{(bi + 1) * page - 1} lies in a block shared with another "
                                   f"request: a session that went back behind a fork point cannot write there")
        first = self.e.prefill(self.slot, tokens, start_pos=self.position)
        self.tokens += tokens
        self.pending = int(first.item()) if hasattr(first, "item") else int(first)
        return self.pending

    def step(self, token: Optional[int] = None) -> int:
        """Feeds one token (default: the pending pick) -> the next pick."""
        if token is None:
            if self.pending is None:
                raise ValueError("nothing pending: feed a prompt first")
            token = self.pending
        return self.feed([token])

    def generate(self, n: int, stop: Sequence[int] = ()) -> List[int]:
        """Greedy continuation: up to `n` tokens, each fed behind the cursor as it is emitted (a stop token is emitted
        and not fed); the pick after the last fed token stays pending, so calls compose."""
        out: List[int] = []
        for _ in range(n):
            t = self.pending
            if t is None:
                raise ValueError("nothing pending: feed a prompt first")
            out.append(t)
            if t in stop:
                break
            self.step()
        return out

    def checkpoint(self) -> int:
        return self.position

    def rollback(self, position: int) -> None:
        """Moves the cursor back to `position` (0 <= position <= current).  The pick after that position is unknown
        until something is fed again (unless the cursor did not move)."""
        if not 0 <= position <= self.position:
            raise ValueError(f"rollback to {position} outside 0..{self.position}")
        if position == self.position:
            return
        del self.tokens[position:]
        self.e.lengths[self.slot] = position
        self.pending = None

    def fork(self, slot: int) -> "Session":
        """A second session in `slot` that continues from this cursor: full blocks are shared, the rest is fed again."""
        if slot == self.slot:
            raise ValueError("fork needs another slot")
        other = Session(self.e, slot)
        page = self.e.kv.page
        full = self.position // page
        if full:
            self.e.kv.attach(slot, list(self.e.kv.req_blocks[self.slot][:full]))
            other.tokens = list(self.tokens[:full * page])
            self.e.lengths[slot] = full * page
        rest = self.tokens[full * page:]
        if rest:
            other.feed(rest)
        else:
            other.pending = self.pending
        return other

    def close(self) -> None:
        self.e.kv.release(self.slot)
        self.e.lengths[self.slot] = 0
        self.tokens, self.pending = [], None
