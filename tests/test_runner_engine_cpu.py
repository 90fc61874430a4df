"""Generic runner adapter behind the scheduler, with a host-side toy runner: concurrent requests get the tokens the
runner gives one request at a time, no prefix is ever reused, blocks return to the table."""
import torch

from dgpp_b200.engine.adapters import RunnerEngine
from dgpp_b200.runtime import rt


class ToyRunner:
    """Next token = (sum of the request's tokens so far * 31 + length) mod vocab: any state mix-up changes the output."""

    def __init__(self, slots, vocab=97):
        self.vocab, self.lengths, self.acc, self.dev = vocab, [0] * slots, [0] * slots, "cpu"
        self.resets = 0

    def _logits(self, slot):
        out = torch.zeros(1, self.vocab)
        out[0, (self.acc[slot] * 31 + self.lengths[slot]) % self.vocab] = 1.0
        return out

    def reset(self, slot):
        self.lengths[slot], self.acc[slot] = 0, 0
        self.resets += 1

    def prefill(self, slot, tokens, chunk=64):
        for t in tokens:
            self.acc[slot] += t
            self.lengths[slot] += 1
        return self._logits(slot)

    def decode(self, slots, tokens):
        rows = []
        for s, t in zip(slots, tokens):
            self.acc[s] += t
            self.lengths[s] += 1
            rows.append(self._logits(s))
        return torch.cat(rows)


def _alone(prompt, n):
    r = ToyRunner(1)
    tok = int(torch.argmax(r.prefill(0, prompt)))
    out = [tok]
    for _ in range(n - 1):
        tok = int(torch.argmax(r.decode([0], [tok])))
        out.append(tok)
    return out


def test_concurrent_requests_match_single_request_runs_and_never_share_a_prefix():
    g = torch.Generator().manual_seed(1)
    shared = torch.randint(0, 97, (200,), generator=g).tolist()
    reqs = {f"r{i}": shared + torch.randint(0, 97, (5 + 7 * i,), generator=g).tolist() for i in range(5)}
    for cache in (True, False):
        runner = ToyRunner(slots=3)
        eng = RunnerEngine(runner, max_context=512, block_tokens=16, prefill_chunk=64)
        sc = rt.SchedulerConfig()
        sc.prefix_cache = cache
        sc.prefix_min_tokens = 16
        s = rt.Scheduler(eng, sc)
        free0 = eng.free_blocks()
        for rid, p in reqs.items():
            s.submit(rid, p, 9)
        s.run(100000)
        got = {}
        for kind, x, a, b in s.events():
            if kind == "token":
                got.setdefault(x, []).append(a)
        assert got == {rid: _alone(p, 9) for rid, p in reqs.items()}, cache
        assert s.meters()["prefix_hit_tokens"] == 0 and eng.usable_prefix([1, 2, 3]) == 0
        assert runner.resets >= 5
        if not cache:                                            # (with the cache on, published blocks stay retained by it)
            assert eng.free_blocks() == free0
        assert not eng.reserve(0, 512 + 16 * 2)                  # beyond the per-request table
