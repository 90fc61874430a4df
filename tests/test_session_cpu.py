"""Session cursor on CPU against an oracle-backed row engine: piecewise feeding, stepping, rollback, fork."""
import pytest
import torch

from dgpp_b200.engine.kv_cache import PagedKV
from dgpp_b200.engine.session import Session
from dgpp_b200.models.dense import DenseConfig, DenseModel


class OracleRows:
    """The engine shape a Session needs, computed by the dense oracle.  What a position holds is stored per PHYSICAL
    block, like KV: a slot that shares blocks with another one sees the tokens the other one wrote there."""

    def __init__(self, model, slots=3, max_seq_len=256, page=16):
        self.m, self.lengths = model, [0] * slots
        c = model.cfg
        self.kv = PagedKV(1, c.kv_heads, c.head_dim, slots * (max_seq_len // page + 1), slots, max_seq_len // page + 1, page,
                          False, "cpu")
        self.store = {}                      # physical block -> list of token ids
        self.calls = 0

    def prefill(self, slot, tokens, start_pos=0):
        assert self.kv.reserve(slot, start_pos + len(tokens))
        self.calls += 1
        page, blocks = self.kv.page, self.kv.req_blocks[slot]
        for i, t in enumerate(tokens):
            p = start_pos + i
            self.store.setdefault(blocks[p // page], [0] * page)[p % page] = int(t)
        toks = [self.store[blocks[p // page]][p % page] for p in range(start_pos + len(tokens))]
        logits, _ = self.m.forward_reference(torch.tensor(toks))
        self.lengths[slot] = len(toks)
        return torch.argsort(-logits[-1].float(), stable=True)[:1].to(torch.int32)


@pytest.fixture(scope="module")
def eng():
    cfg = DenseConfig.tiny(vocab=512, weight_fmt="bf16")
    return OracleRows(DenseModel.random_init(cfg, device="cpu", seed=3, std=0.05))


def _greedy(model, toks, n):
    cur, out = list(toks), []
    for _ in range(n):
        lg, _ = model.forward_reference(torch.tensor(cur))
        t = int(torch.argsort(-lg[-1].float(), stable=True)[0])
        out.append(t)
        cur.append(t)
    return out


def test_piecewise_feed_step_and_generate(eng):
    p = torch.randint(0, 512, (37,), generator=torch.Generator().manual_seed(0)).tolist()
    s = Session(eng, 0)
    s.feed(p[:5])
    s.feed(p[5:30])
    first = s.feed(p[30:])
    want = _greedy(eng.m, p, 6)
    assert s.position == 37 and first == want[0]
    # every emitted token is fed behind the cursor; the pick after the last one stays pending
    assert s.generate(5) == want[:5] and s.position == 37 + 5 and s.pending == want[5]
    with pytest.raises(ValueError):
        s.feed([])
    s.close()
    assert s.position == 0 and eng.kv.req_blocks[0] == []


def test_rollback_and_fork(eng):
    p = torch.randint(0, 512, (40,), generator=torch.Generator().manual_seed(1)).tolist()
    s = Session(eng, 0)
    s.feed(p)
    mark = s.checkpoint()
    a = s.generate(4)
    s.rollback(mark)
    assert s.position == 40 and s.pending is None and eng.lengths[0] == 40
    # another continuation from the same prefix, then the original one again
    other = (a[0] + 1) % 512
    nxt = s.feed([other])
    lg, _ = eng.m.forward_reference(torch.tensor(p + [other]))
    assert nxt == int(torch.argsort(-lg[-1].float(), stable=True)[0])
    s.rollback(mark)
    s.feed([a[0]])
    assert s.generate(3) == a[1:4]
    with pytest.raises(ValueError):
        s.rollback(1000)
    # fork: full blocks shared by reference, the remainder fed again; both continue alike
    s.rollback(mark)
    s.feed(p[:3])                                   # position 43: two full blocks of 16 + 11 tokens
    f = s.fork(1)
    assert f.position == s.position == 43 and f.pending == s.pending
    shared = eng.kv.req_blocks[0][:2]
    assert eng.kv.req_blocks[1][:2] == shared and all(eng.kv.alloc.refcount(b) == 2 for b in shared)
    assert f.generate(3) == s.generate(3)
    # going back behind the fork point and writing there would change what the fork reads: refused
    s.rollback(10)
    with pytest.raises(RuntimeError, match="shared"):
        s.feed([1, 2, 3])
    f.close()
    assert s.feed([1, 2, 3]) >= 0                   # the blocks are this session's alone again
    assert all(eng.kv.alloc.refcount(b) == 1 for b in shared)
    with pytest.raises(ValueError):
        s.fork(0)
    s.close()
