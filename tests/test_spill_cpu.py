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
    key = eng.key(rt.chain_hash(rt.FNV_SEED, A[:16]))
    assert tier.contains(key) and tier.corrupt_for_test(key)
    again, _ = _run(eng, [("a2", A)], prefix_cache=True)
    assert again["a2"] == first["a1"] and tier.stats()["crc_failures"] == 1


def test_adopted_tier_of_another_model_gives_no_hits(tmp_path):
    """A tier directory reopened by an engine with another fingerprint (other weights, quantisation, shard ...) must
    not hand back the blocks the first engine spilled, although tokens and page geometry are the same."""
    from dgpp_b200.engine.spill import cache_fingerprint, weights_digest

    mcfg = DenseConfig.plumbing_fp32()
    g = torch.Generator().manual_seed(3)
    A = torch.randint(0, mcfg.vocab, (70,), generator=g).tolist()
    B = torch.randint(0, mcfg.vocab, (66,), generator=g).tolist()

    def engine(seed):
        model = DenseModel.random_init(mcfg, device="cpu", seed=seed)
        inner = Counting(model, slots=1, num_blocks=8, block_tokens=16, max_context=256)
        tier = rt.DiskTier(str(tmp_path), page_bytes=1 << 16, pages=64)          # adopts what is there
        fp = cache_fingerprint(config=mcfg.name, weights=weights_digest([L.qkv.payload for L in model.layers]),
                               kv="fp32", tp=(0, 1))
        return SpillingEngine(inner, tier, fingerprint=fp), tier, inner

    e0, t0, _ = engine(0)
    _run(e0, [("a1", A), ("b1", B)], prefix_cache=True)
    t0.flush()
    t0.commit()
    assert e0.spilled >= 4
    del e0, t0
    # same weights: the adopted blocks are found
    e1, t1, i1 = engine(0)
    assert t1.blobs() >= 4
    _run(e1, [("a2", A)], prefix_cache=True)
    assert e1.restored == 4
    t1.flush()
    t1.commit()
    del e1, t1
    # other weights, same tokens, same geometry: nothing may be restored
    e2, t2, i2 = engine(1)
    _run(e2, [("a3", A)], prefix_cache=True)
    assert e2.restored == 0 and i2.computed >= len(A)
