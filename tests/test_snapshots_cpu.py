"""Snapshot table of the hybrid engine (CPU, fakes in place of the kernel runner): eviction when the table is full
and some entries are dead must not fail while it drops them."""
from dgpp_b200.engine.adapters import HybridEngine


class _Alloc:
    def __init__(self):
        self.gen, self.ref = {}, {}

    def generation(self, b):
        return self.gen.get(b, 0)

    def refcount(self, b):
        return self.ref.get(b, 0)


class _KV:
    page = 16

    def __init__(self):
        self.alloc = _Alloc()
        self.req_blocks = {0: list(range(100))}


class _Runner:
    def __init__(self):
        self.kv = _KV()
        self.lengths = [0]
        self.gdn_state = {}


def test_full_snapshot_table_with_dead_entries_is_pruned_not_raised():
    eng = HybridEngine(_Runner(), snapshot_every=16, max_snapshots=2)
    kv = eng.kv
    for b in range(100):
        kv.alloc.ref[b] = 1
    eng._snapshot(0, 16)                    # block 0
    eng._snapshot(0, 32)                    # block 1: table full
    kv.alloc.ref[1] = 0                     # block 1 is freed: its snapshot is dead (and it is the LAST key)
    eng._snapshot(0, 48)                    # used to raise "dictionary changed size during iteration"
    assert set(eng.snaps) == {0, 2}
    kv.alloc.gen[0] = 7                     # block 0 recycled: generation mismatch -> dead
    eng._snapshot(0, 64)
    assert set(eng.snaps) == {2, 3}
    eng._snapshot(0, 80)                    # nothing dead: the oldest live entry goes
    assert set(eng.snaps) == {3, 4} and eng.snapshots_taken == 5
    assert eng.usable_prefix([9, 3]) == 2 and eng.usable_prefix([9, 8]) == 0
