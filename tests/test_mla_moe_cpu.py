"""MLA + MoE family oracle on CPU: causal consistency, and the sparse index degenerates to dense attention when it
keeps every position."""
import torch

from dgpp_b200.models.mla_moe import MlaMoeConfig, MlaMoeModel


def test_oracle_is_causal_and_full_topk_equals_dense():
    cfg = MlaMoeConfig(layers=2, hidden=256, heads=4, q_lora=64, kv_lora=64, nope=32, rope=16, v_dim=32, ffn=512,
                       vocab=512, index_heads=2, index_dim=32, index_topk=1000)
    m = MlaMoeModel.random_init(cfg, "cpu", seed=1, std=0.05)
    toks = torch.randint(0, cfg.vocab, (40,))
    full = m.forward_reference(toks)
    # causal: the logits of the first 25 positions do not depend on later tokens
    part = m.forward_reference(toks[:25])
    assert torch.allclose(full[:25], part, atol=1e-5)
    # the index keeps everything -> same as a model without an index
    for L in m.layers:
        L.idx_q = L.idx_k = L.idx_w = None
    dense = m.forward_reference(toks)
    assert torch.equal(dense, full)
    # a small top-k changes the result for long enough contexts only
    m2 = MlaMoeModel.random_init(MlaMoeConfig(**{**cfg.__dict__, "index_topk": 8}), "cpu", seed=1, std=0.05)
    sparse = m2.forward_reference(toks)
    assert torch.allclose(sparse[:8], full[:8], atol=1e-5) and (sparse[20:] - full[20:]).abs().max() > 1e-4
