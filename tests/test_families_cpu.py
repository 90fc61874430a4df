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
