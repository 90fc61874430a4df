"""Hashed n-gram memory on CPU: the hash against plain Python integers, the lookback chaining across chunks, the gate,
and the sites inside the stream family's oracle."""
import math

import torch

from dgpp_b200.models.engram import Engram, EngramConfig
from dgpp_b200.models.glm_flash import GlmFlashConfig, GlmFlashModel
from dgpp_b200.ops import reference as ref


def _wrap(v):                      # two's-complement 64-bit
    v &= (1 << 64) - 1
    return v - (1 << 64) if v >= (1 << 63) else v


def test_hash_matches_python_integers_and_lookback_chains():
    cfg = EngramConfig(max_ngram=4, heads=2, head_dim=64, bucket=500)
    e = Engram.random_init(cfg, [0], 300, 4, 128, "cpu", seed=3)
    L = e.layers[0]
    # large multipliers so that the products wrap
    L.multipliers = torch.tensor([0x7123456789ABCDE1, 0x6FEDCBA987654321, 0x5555555555555555, 0x7777777777777771], dtype=torch.int64)
    toks = torch.randint(0, 300, (9,), generator=torch.Generator().manual_seed(1), dtype=torch.int32)
    prev = torch.tensor(e.prev_rows(toks.tolist(), []), dtype=torch.int32)
    assert prev[0].tolist() == [-1] + toks[:-1].tolist() and prev[2, :3].tolist() == [-1, -1, -1]
    ids = ref.engram_ids(toks, prev, e.token_map, L.multipliers, L.primes, L.offsets, e.pad_class)
    assert ids.shape == (9, 6)
    tm, mult = e.token_map.tolist(), L.multipliers.tolist()
    for t in range(9):
        y = [tm[int(toks[t])]] + [tm[int(toks[t - k])] if t - k >= 0 else e.pad_class for k in range(1, 4)]
        rolling = _wrap(y[0] * mult[0])
        for n in range(1, 4):
            rolling = _wrap(rolling ^ _wrap(y[n] * mult[n]))
            for h in range(2):
                prime = int(L.primes[n - 1, h])
                assert int(ids[t, (n - 1) * 2 + h]) == rolling % prime + int(L.offsets[n - 1, h])
    assert int(ids.min()) >= 0 and int(ids.max()) < L.table.shape[0]
    # a later chunk continues the lookback from the kept history
    hist = e.keep([], toks[:5].tolist())
    assert hist == toks[2:5].tolist()
    tail = torch.tensor(e.prev_rows(toks[5:].tolist(), hist), dtype=torch.int32)
    assert torch.equal(tail, prev[:, 5:])
    # rows decode exactly: e4m3 value times a power of two
    emb = ref.engram_embed(toks, prev, e.token_map, L.multipliers, L.primes, L.offsets, L.table, L.table_sf, e.pad_class)
    row = L.table[ids[4, 3]].view(torch.float8_e4m3fn).float() * torch.exp2(L.table_sf[ids[4, 3]].float() - 127).repeat_interleave(32)
    assert torch.equal(emb[4, 3 * 64:4 * 64].float(), row)


def test_gate_formula():
    g = torch.Generator().manual_seed(2)
    x = torch.randn(5, 4, 128, generator=g).to(torch.bfloat16)
    kv = torch.randn(5, 5 * 128, generator=g).to(torch.bfloat16)
    qw, kw = torch.randn(4, 128, generator=g).to(torch.bfloat16), torch.randn(4, 128, generator=g).to(torch.bfloat16)
    out = ref.engram_gate(x, kv, qw, kw, 1e-6).float()
    t, i = 3, 2
    xi, key, val = x[t, i].float(), kv[t, i * 128:(i + 1) * 128].float(), kv[t, 4 * 128:].float()
    dot = float((xi * qw[i].float() * kw[i].float() * key).sum()) / math.sqrt(float(xi.pow(2).mean()) + 1e-6) \
        / math.sqrt(float(key.pow(2).mean()) + 1e-6) / math.sqrt(128)
    gate = 1 / (1 + math.exp(-math.copysign(math.sqrt(max(abs(dot), 1e-6)), dot)))
    assert torch.allclose(out[t, i], (xi + gate * val).to(torch.bfloat16).float(), atol=2e-2)
    assert 0.0 < gate < 1.0


def test_sites_in_the_stream_family_are_causal_and_local():
    cfg = GlmFlashConfig(layers=4, hidden=256, vocab=512, mla_every=2, k_heads=2, v_heads=2, dk=64, dv=64, heads=4,
                         q_lora=128, kv_lora=64, nope=32, rope=32, v_dim=32, ffn=512, engram=EngramConfig(bucket=300),
                         engram_layers=(1, 3))
    m = GlmFlashModel.random_init(cfg, "cpu", seed=1)
    assert sorted(m.engram.layers) == [1, 3]
    t = torch.randint(0, 512, (14,), generator=torch.Generator().manual_seed(0))
    full = m.forward_reference(t)
    plain = GlmFlashModel.random_init(GlmFlashConfig(**{**cfg.__dict__, "engram": None}), "cpu", seed=1)
    assert (plain.forward_reference(t) - full).abs().max().item() > 1e-2
    t2 = t.clone()
    t2[9] = (t2[9] + 1) % 512
    diff = (m.forward_reference(t2) - full).abs().max(1).values
    assert diff[:9].max().item() == 0.0 and diff[9:].min().item() > 0.0
