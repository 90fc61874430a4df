"""Family oracles on CPU: causality, loop / branch bookkeeping, the hashed bigram ids."""
import torch

from dgpp_b200.models.dory import DoryConfig, DoryModel
from dgpp_b200.models.flash_next import FlashNextConfig, FlashNextModel


def test_dory_oracle_is_causal_and_loops_change_the_result():
    cfg = DoryConfig(hidden=256, head_dim=64, ffn=512, vocab=512, loops=2)
    m = DoryModel.random_init(cfg, "cpu", seed=1)
    t = torch.randint(0, 512, (12,), generator=torch.Generator().manual_seed(0))
    full = m.forward_reference(t)
    t2 = t.clone()
    t2[8] = (t2[8] + 3) % 512
    diff = (m.forward_reference(t2) - full).abs().max(1).values
    assert diff[:8].max().item() == 0.0 and diff[8:].min().item() > 0.0
    m.cfg = DoryConfig(**{**cfg.__dict__, "loops": 3})
    assert (m.forward_reference(t) - full).abs().max().item() > 1e-3


def test_flash_next_oracle_is_causal_and_bigram_ids_chain():
    cfg = FlashNextConfig(layers=4, hidden=256, full_every=2, q_heads=4, kv_heads=2, head_dim=64, gdn_k_heads=2, gdn_v_heads=2,
                          gdn_dk=64, gdn_dv=64, ffn=512, vocab=512, gr_rank=64, ple_rows=128)
    m = FlashNextModel.random_init(cfg, "cpu", seed=1)
    t = torch.randint(0, 512, (12,), generator=torch.Generator().manual_seed(0))
    full = m.forward_reference(t)
    t2 = t.clone()
    t2[9] = (t2[9] + 5) % 512
    diff = (m.forward_reference(t2) - full).abs().max(1).values
    assert diff[:9].max().item() == 0.0 and diff[9:].min().item() > 0.0
    ids = m.ple_ids(t.tolist())
    assert ids[0] == cfg.ple_id(0, int(t[0])) and ids[5] == cfg.ple_id(int(t[4]), int(t[5]))
    assert m.ple_ids(t[6:].tolist(), prev=int(t[5])) == ids[6:]          # a later chunk continues the chain


def test_flash_next_pooled_key_sparse_attention_oracle():
    import math

    from dgpp_b200.models.flash_next import QsaConfig, qsa_keep_reference
    from dgpp_b200.ops import reference as ref

    # the kept set against a direct restatement: complete visible blocks by score, own incomplete block on top
    g = torch.Generator().manual_seed(4)
    T, ih, di, page, k = 45, 2, 32, 8, 2
    iq, raw = torch.randn(T, ih, di, generator=g), torch.randn(T, di, generator=g).to(torch.bfloat16).float()
    kn = (0.1 * torch.randn(di, generator=g)).to(torch.bfloat16)
    inv, _ = ref.rope_inv_freq(di, 1e4, "cpu")
    keep = qsa_keep_reference(iq, raw, kn, inv, page, k, 1e-6)
    comp = []
    for b in range(T // page):
        mean = ref._r(raw[b * page:(b + 1) * page].mean(0, keepdim=True))
        comp.append(ref.apply_rope(ref.head_norm(mean.unsqueeze(1), kn, 1e-6, True), torch.tensor([b * page]), inv, di)[0, 0])
    for t in range(T):
        vis = (t + 1) // page
        sc = [float(torch.relu(iq[t] @ comp[b]).sum()) / math.sqrt(di) for b in range(vis)]
        want = set(sorted(range(vis), key=lambda b: (-sc[b], b))[:k])
        if (t + 1) % page:
            want.add(t // page)
        assert set(torch.nonzero(keep[t]).flatten().tolist()) == want, t
    assert keep[7].tolist()[:1] == [True] and int(keep[44].sum()) == 3

    cfg = FlashNextConfig(layers=2, hidden=256, full_every=2, q_heads=4, kv_heads=2, head_dim=64, gdn_k_heads=2, gdn_v_heads=2,
                          gdn_dk=64, gdn_dv=64, ffn=512, vocab=512, gr_rank=64, ple_rows=0, page=8,
                          qsa=QsaConfig(index_heads=2, index_dim=64, select_k=1))
    m = FlashNextModel.random_init(cfg, "cpu", seed=2)
    t = torch.randint(0, 512, (40,), generator=torch.Generator().manual_seed(0))
    full = m.forward_reference(t)
    t2 = t.clone()
    t2[33] = (t2[33] + 5) % 512
    diff = (m.forward_reference(t2) - full).abs().max(1).values
    assert diff[:33].max().item() == 0.0 and diff[33:].min().item() > 0.0
    # keeping every block gives another result from position 2 * page on: the selection really drops tokens
    m.cfg.qsa.select_k = 64
    every = m.forward_reference(t)
    assert torch.equal(every[:15], full[:15]) and (every[24:] - full[24:]).abs().max().item() > 1e-4
