"""KV cold tier on CPU: blocks evicted from a small pool are spilled to the disk tier and restored byte for byte at
a later prefill; tokens equal those of an engine without the tier, and fewer prompt tokens are recomputed."""
import torch

from dgpp_b200.engine.adapters import ReferenceEngine
from dgpp_b200.engine.spill import SpillingEngine
from dgpp_b200.models.dense import DenseConfig, DenseModel
from dgpp_b200.runtime import rt


class Counting(ReferenceEngine):
    computed = 0

    def prefill(self, slot, tokens, pos, last):
        self.computed += len(tokens)
        return super().prefill(slot, tokens, pos, last)


def _run(engine, reqs, prefix_cache):
    cfg = rt.SchedulerConfig()
    cfg.prefix_cache = prefix_cache
    cfg.prefix_min_tokens = 16
    s = rt.Scheduler(engine, cfg)
    out = {}
    for rid, p in reqs:                                  # strictly one after the other
        s.submit(rid, p, 5)
        s.run(100000)
        for kind, r, a, b in s.events():
            if kind == "token":
                out.setdefault(r, []).append(a)
    return out, s.meters()


def test_spill_and_restore_round_trip(tmp_path):
    mcfg = DenseConfig.plumbing_fp32()
    model = DenseModel.random_init(mcfg, device="cpu", seed=0)
    g = torch.Generator().manual_seed(3)
    A = torch.randint(0, mcfg.vocab, (70,), generator=g).tolist()
    B = torch.randint(0, mcfg.vocab, (66,), generator=g).tolist()
    reqs = [("a1", A), ("b1", B), ("a2", A + [5, 6, 7])]
    # baseline: no prefix cache, no tier
    base = Counting(model, slots=1, num_blocks=8, block_tokens=16, max_context=256)
    want, _ = _run(base, reqs, prefix_cache=False)
    # a pool of 8 blocks cannot keep A's 4 cached blocks while B (5 blocks) runs: the prefix cache evicts them, the
    # wrapper spills them, and a2 finds nothing in memory but everything on disk
    inner = Counting(model, slots=1, num_blocks=8, block_tokens=16, max_context=256)
    tier = rt.DiskTier(str(tmp_path), page_bytes=1 << 16, pages=64)
    eng = SpillingEngine(inner, tier)
    got, m = _run(eng, reqs, prefix_cache=True)
    tier.flush()
    assert got == want
    assert eng.spilled >= 4 and eng.restored == 4 and eng.restored_tokens == 64
    assert inner.computed == base.computed - 64          # a2 recomputed only what follows the restored blocks
    assert tier.stats()["crc_failures"] == 0


def test_corrupted_page_falls_back_to_computing(tmp_path):
    mcfg = DenseConfig.plumbing_fp32()
    model = DenseModel.random_init(mcfg, device="cpu", seed=0)
    g = torch.Generator().manual_seed(4)
    A = torch.randint(0, mcfg.vocab, (40,), generator=g).tolist()
    B = torch.randint(0, mcfg.vocab, (100,), generator=g).tolist()
    inner = Counting(model, slots=1, num_blocks=8, block_tokens=16, max_context=256)
    tier = rt.DiskTier(str(tmp_path), page_bytes=1 << 16, pages=64)
    eng = SpillingEngine(inner, tier)
    first, _ = _run(eng, [("a1", A), ("b1", B)], prefix_cache=True)
    tier.flush()
    key = rt.chain_hash(rt.FNV_SEED, A[:16])
    assert tier.contains(key) and tier.corrupt_for_test(key)
    again, _ = _run(eng, [("a2", A)], prefix_cache=True)
    assert again["a2"] == first["a1"] and tier.stats()["crc_failures"] == 1
